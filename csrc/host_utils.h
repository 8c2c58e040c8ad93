// Host-side helpers shared by the launchers: TMA tensor-map encoding through the driver
// entry point (no link-time dependency on libcuda), error strings, SM count.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

namespace axb {

// Return codes of the extern "C" launchers. 0 = launched; negative = refused before launch.
enum : int {
  AXB_LAUNCH_OK = 0,
  AXB_LAUNCH_BAD_ARG = -1,
  AXB_LAUNCH_NO_DRIVER = -2,
  AXB_LAUNCH_TMAP_FAILED = -3,
  AXB_LAUNCH_CUDA_ERROR = -4,
  AXB_LAUNCH_TOO_LARGE = -5,
};

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn get_encode_tiled() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) ==
            cudaSuccess &&
        q == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeTiledFn>(p);
    }
  }
  return fn;
}

// 2-D row-major tensor [outer][inner] with a row pitch in bytes; box = [box_outer][box_inner].
// swizzle128 = true gives CU_TENSOR_MAP_SWIZZLE_128B (box_inner * elem must be 128 bytes).
inline int make_tmap_2d(CUtensorMap* out, const void* base, CUtensorMapDataType dt,
                        int elem_bytes, uint64_t inner, uint64_t outer, uint64_t pitch_bytes,
                        uint32_t box_inner, uint32_t box_outer, bool swizzle128) {
  EncodeTiledFn enc = get_encode_tiled();
  if (enc == nullptr) return AXB_LAUNCH_NO_DRIVER;
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || (pitch_bytes & 15) != 0)
    return AXB_LAUNCH_BAD_ARG;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {pitch_bytes};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(out, dt, 2, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE,
                   swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  (void)elem_bytes;
  return r == CUDA_SUCCESS ? AXB_LAUNCH_OK : AXB_LAUNCH_TMAP_FAILED;
}

// 3-D tensor [d2][d1][d0] (d0 innermost) with byte pitches for d1 and d2.
inline int make_tmap_3d(CUtensorMap* out, const void* base, CUtensorMapDataType dt, uint64_t d0,
                        uint64_t d1, uint64_t d2, uint64_t pitch1_bytes, uint64_t pitch2_bytes,
                        uint32_t b0, uint32_t b1, uint32_t b2, bool swizzle128) {
  EncodeTiledFn enc = get_encode_tiled();
  if (enc == nullptr) return AXB_LAUNCH_NO_DRIVER;
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || (pitch1_bytes & 15) != 0 ||
      (pitch2_bytes & 15) != 0)
    return AXB_LAUNCH_BAD_ARG;
  cuuint64_t dims[3] = {d0, d1, d2};
  cuuint64_t strides[2] = {pitch1_bytes, pitch2_bytes};
  cuuint32_t box[3] = {b0, b1, b2};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(out, dt, 3, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE,
                   swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? AXB_LAUNCH_OK : AXB_LAUNCH_TMAP_FAILED;
}

inline int sm_count() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 148;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
      n = 148;
  }
  return n;
}

// Launch as a programmatic dependent of the previous kernel of the stream: the grid may be scheduled while that
// kernel drains, so launch latency and CTA ramp-up overlap its tail. The kernel MUST execute griddepcontrol.wait
// (grid_dependency_wait) before its first global memory access; only kernels written that way are launched here.
template <typename... KArgs, typename... Args>
inline int launch_dependent(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...) != cudaSuccess) {
    cudaGetLastError();
    return -4;   // AXB_LAUNCH_CUDA_ERROR
  }
  return 0;
}

inline int check_launch() {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    fprintf(stderr, "[axon_b200] kernel launch failed: %s\n", cudaGetErrorString(e));
    return AXB_LAUNCH_CUDA_ERROR;
  }
  return AXB_LAUNCH_OK;
}

}  // namespace axb
