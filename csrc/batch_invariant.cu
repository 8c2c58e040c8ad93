// Row-wise log-softmax and mean whose result for a row never depends on how many rows are in the
// batch: one block per row, a fixed number of threads, fixed-order tree reductions. Together with
// the fixed-configuration GEMM path (no split-K, one tile width) they give a sampler whose
// log-probs for a request do not change with the requests it happens to be batched with.
#include "host_utils.h"
#include "ptx.cuh"

namespace axb {

constexpr int BI_THREADS = 256;

__device__ __forceinline__ float block_reduce_max(float v, float* red) {
  v = warp_max(v);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float r = red[0];
#pragma unroll
  for (int i = 1; i < BI_THREADS / 32; ++i) r = fmaxf(r, red[i]);
  __syncthreads();
  return r;
}
__device__ __forceinline__ float block_reduce_sum(float v, float* red) {
  v = warp_sum(v);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float r = 0.f;
#pragma unroll
  for (int i = 0; i < BI_THREADS / 32; ++i) r += red[i];
  __syncthreads();
  return r;
}

template <class T>
__device__ __forceinline__ float ldf(const T* p, long long i);
template <>
__device__ __forceinline__ float ldf<float>(const float* p, long long i) { return p[i]; }
template <>
__device__ __forceinline__ float ldf<__nv_bfloat16>(const __nv_bfloat16* p, long long i) { return __bfloat162float(p[i]); }

template <class T>
__global__ void __launch_bounds__(BI_THREADS) log_softmax_rows_kernel(const T* __restrict__ x, float* __restrict__ out,
                                                                       int cols, long long ldx) {
  __shared__ float red[BI_THREADS / 32];
  const long long r = blockIdx.x;
  const T* row = x + r * ldx;
  float mx = -INFINITY;
  for (int c = threadIdx.x; c < cols; c += BI_THREADS) mx = fmaxf(mx, ldf(row, c));
  mx = block_reduce_max(mx, red);
  float s = 0.f;
  for (int c = threadIdx.x; c < cols; c += BI_THREADS) s += expf(ldf(row, c) - mx);
  s = block_reduce_sum(s, red);
  const float lse = mx + logf(s);
  for (int c = threadIdx.x; c < cols; c += BI_THREADS) out[r * cols + c] = ldf(row, c) - lse;
}

template <class T>
__global__ void __launch_bounds__(BI_THREADS) mean_rows_kernel(const T* __restrict__ x, float* __restrict__ out, int cols,
                                                               long long ldx) {
  __shared__ float red[BI_THREADS / 32];
  const long long r = blockIdx.x;
  float s = 0.f;
  for (int c = threadIdx.x; c < cols; c += BI_THREADS) s += ldf(x + r * ldx, c);
  s = block_reduce_sum(s, red);
  if (threadIdx.x == 0) out[r] = s / cols;
}

}  // namespace axb

using namespace axb;

extern "C" int axb_log_softmax_rows(const void* x, int is_bf16, float* out, long long rows, int cols, long long ldx,
                                    void* stream) {
  if (rows <= 0 || cols <= 0 || rows > 0x7fffffffLL) return AXB_LAUNCH_BAD_ARG;
  cudaStream_t s = (cudaStream_t)stream;
  if (is_bf16) log_softmax_rows_kernel<__nv_bfloat16><<<(int)rows, BI_THREADS, 0, s>>>((const __nv_bfloat16*)x, out, cols, ldx);
  else log_softmax_rows_kernel<float><<<(int)rows, BI_THREADS, 0, s>>>((const float*)x, out, cols, ldx);
  return check_launch();
}

extern "C" int axb_mean_rows(const void* x, int is_bf16, float* out, long long rows, int cols, long long ldx, void* stream) {
  if (rows <= 0 || cols <= 0 || rows > 0x7fffffffLL) return AXB_LAUNCH_BAD_ARG;
  cudaStream_t s = (cudaStream_t)stream;
  if (is_bf16) mean_rows_kernel<__nv_bfloat16><<<(int)rows, BI_THREADS, 0, s>>>((const __nv_bfloat16*)x, out, cols, ldx);
  else mean_rows_kernel<float><<<(int)rows, BI_THREADS, 0, s>>>((const float*)x, out, cols, ldx);
  return check_launch();
}
