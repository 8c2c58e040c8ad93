// Device-side index checks for the debug build (-DAXB_DEBUG).
//
// A release kernel that meets an index outside its buffers clamps or skips it silently (the access never
// happens). The debug build additionally RECORDS the first such index: AXB_DEBUG_CHECK(cond, a, b) writes
// {AXB_ERR_BAD_ARG, source line, a, b} into a small device array when `cond` is false and lets the kernel
// carry on with its skip / clamp path. Nothing traps, nothing faults; the host reads the record with
// axb_debug_status() after a synchronise. The array is per translation unit (no relocatable device code is
// needed); every unit that uses the macro registers a reader with the collector in debug.cu.
#pragma once
#include <cuda_runtime.h>

#ifdef AXB_DEBUG
namespace axb_dbg {
void register_reader(int (*reader)(int*), const char* file);      // debug.cu

static __device__ int word[4];

static int read_and_clear(int* out4) {
  if (cudaMemcpyFromSymbol(out4, word, 16) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  if (out4[0] != 0) {
    const int zero[4] = {0, 0, 0, 0};
    cudaMemcpyToSymbol(word, zero, 16);
  }
  return out4[0];
}

namespace {
struct Registrar {
  Registrar() { register_reader(&read_and_clear, __BASE_FILE__); }   // the unit being compiled, not this header
};
static Registrar registrar;
}  // namespace

__device__ __forceinline__ void record(int line, long long a, long long b) {
  if (atomicCAS(&word[0], 0, 6 /* AXB_ERR_BAD_ARG */) == 0) {
    word[1] = line;
    word[2] = (int)a;
    word[3] = (int)b;
  }
}
}  // namespace axb_dbg
#define AXB_DEBUG_CHECK(cond, a, b)                          \
  do {                                                       \
    if (!(cond)) axb_dbg::record(__LINE__, (long long)(a), (long long)(b)); \
  } while (0)
#else
#define AXB_DEBUG_CHECK(cond, a, b) \
  do {                              \
  } while (0)
#endif
