// Device memory that another PROCESS on the same node can map: plain cudaMalloc allocations exported and
// opened through CUDA IPC handles. The disaggregated weight push uses it: every sampler process keeps
// its live parameter buffer in such an allocation, every trainer process opens the handles once at
// connect time, and from then on the sync-plan kernel stores straight into the samplers' weights over
// NVLink (plain peer stores; no staging copy, no message). Allocations made here do not come from
// PyTorch's caching allocator, whose blocks are sub-allocated and cannot be exported one by one.
#include "host_utils.h"
#include <cstring>

using namespace axb;

extern "C" int axb_ipc_alloc(long long bytes, void** out) {
  if (bytes <= 0 || out == nullptr) return AXB_LAUNCH_BAD_ARG;
  void* p = nullptr;
  if (cudaMalloc(&p, (size_t)bytes) != cudaSuccess) {
    cudaGetLastError();
    return AXB_LAUNCH_CUDA_ERROR;
  }
  *out = p;
  return AXB_LAUNCH_OK;
}

extern "C" int axb_ipc_free(void* p) {
  if (p == nullptr) return AXB_LAUNCH_OK;
  return cudaFree(p) == cudaSuccess ? AXB_LAUNCH_OK : AXB_LAUNCH_CUDA_ERROR;
}

// handle64: 64 bytes written with the opaque IPC handle of the allocation that starts at p.
extern "C" int axb_ipc_export(const void* p, unsigned char* handle64) {
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handles are 64 bytes");
  if (p == nullptr || handle64 == nullptr) return AXB_LAUNCH_BAD_ARG;
  cudaIpcMemHandle_t h;
  if (cudaIpcGetMemHandle(&h, const_cast<void*>(p)) != cudaSuccess) {
    cudaGetLastError();
    return AXB_LAUNCH_CUDA_ERROR;
  }
  memcpy(handle64, &h, 64);
  return AXB_LAUNCH_OK;
}

// Maps another process's allocation into this one (peer access to the owning GPU is enabled by the
// driver on first use). The mapping stays valid until axb_ipc_close or process exit.
extern "C" int axb_ipc_open(const unsigned char* handle64, void** out) {
  if (handle64 == nullptr || out == nullptr) return AXB_LAUNCH_BAD_ARG;
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, 64);
  void* p = nullptr;
  if (cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
    cudaGetLastError();
    return AXB_LAUNCH_CUDA_ERROR;
  }
  *out = p;
  return AXB_LAUNCH_OK;
}

extern "C" int axb_ipc_close(void* p) {
  if (p == nullptr) return AXB_LAUNCH_OK;
  return cudaIpcCloseMemHandle(p) == cudaSuccess ? AXB_LAUNCH_OK : AXB_LAUNCH_CUDA_ERROR;
}
