// Fused optimizer kernels over flat parameter shards: sum of squares (grad norm), clip
// coefficient, and AdamW with fp32 master weights that also emits the bf16 working copy.
// The clip coefficient and the finite flag stay on the device so a step needs no host sync.
#include "ptx.cuh"
#include "host_utils.h"

namespace axb {

constexpr int OPT_THREADS = 256;

// partial[block] = sum g^2 over the block's grid-stride slice. G = float or bf16.
template <class G>
__global__ void __launch_bounds__(OPT_THREADS)
sumsq_kernel(const G* __restrict__ g, long long n, float* __restrict__ partial) {
  __shared__ float red[OPT_THREADS / 32];
  float s = 0.f;
  for (long long i = (long long)blockIdx.x * OPT_THREADS + threadIdx.x; i < n;
       i += (long long)gridDim.x * OPT_THREADS) {
    float v;
    if constexpr (sizeof(G) == 4) v = g[i]; else v = __bfloat162float(g[i]);
    s += v * v;
  }
  s = warp_sum(s);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x < 32) {
    float r = threadIdx.x < OPT_THREADS / 32 ? red[threadIdx.x] : 0.f;
    r = warp_sum(r);
    if (threadIdx.x == 0) partial[blockIdx.x] = r;
  }
}

// out[0] = total sum of squares (fixed-order, deterministic). One block.
__global__ void sumsq_final_kernel(const float* __restrict__ partial, int P, float* __restrict__ out,
                                   int accumulate) {
  __shared__ float red[32];
  float s = 0.f;
  for (int i = threadIdx.x; i < P; i += blockDim.x) s += partial[i];
  s = warp_sum(s);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x < 32) {
    float r = threadIdx.x < blockDim.x / 32 ? red[threadIdx.x] : 0.f;
    r = warp_sum(r);
    if (threadIdx.x == 0) out[0] = accumulate ? out[0] + r : r;
  }
}

// state[0] = total sumsq (input, already reduced across ranks); writes
// state[1] = grad norm, state[2] = clip coefficient (0 when the norm is not finite or above
// skip_threshold), state[3] = 1 if the step must be skipped.
__global__ void clip_coef_kernel(float* state, float max_norm, float skip_threshold, float grad_scale) {
  const float norm = sqrtf(state[0]) * grad_scale;
  const bool finite = isfinite(norm);
  const bool skip = !finite || (skip_threshold > 0.f && norm > skip_threshold);
  float coef = grad_scale;
  if (max_norm > 0.f && finite) coef = grad_scale * fminf(1.f, max_norm / (norm + 1e-6f));
  state[1] = norm;
  state[2] = skip ? 0.f : coef;
  state[3] = skip ? 1.f : 0.f;
}

// AdamW (decoupled weight decay) on a flat shard. state as written by clip_coef_kernel; when
// state == nullptr the gradient is used as is. bc1 = 1 - beta1^t, bc2 = 1 - beta2^t.
template <class G>
__global__ void __launch_bounds__(OPT_THREADS)
adamw_kernel(float* __restrict__ master, __nv_bfloat16* __restrict__ param, const G* __restrict__ grad,
             float* __restrict__ m, float* __restrict__ v, long long n, float lr, float beta1,
             float beta2, float eps, float wd, float bc1, float bc2, const float* __restrict__ state) {
  float coef = 1.f;
  if (state != nullptr) {
    if (state[3] != 0.f) return;
    coef = state[2];
  }
  const float inv_bc1 = 1.f / bc1;
  const float inv_sqrt_bc2 = rsqrtf(bc2);
  for (long long i = (long long)blockIdx.x * OPT_THREADS + threadIdx.x; i < n;
       i += (long long)gridDim.x * OPT_THREADS) {
    float g;
    if constexpr (sizeof(G) == 4) g = grad[i]; else g = __bfloat162float(grad[i]);
    g *= coef;
    const float mi = beta1 * m[i] + (1.f - beta1) * g;
    const float vi = beta2 * v[i] + (1.f - beta2) * g * g;
    m[i] = mi;
    v[i] = vi;
    float p = master[i];
    p -= lr * wd * p;
    p -= lr * (mi * inv_bc1) / (sqrtf(vi) * inv_sqrt_bc2 + eps);
    master[i] = p;
    if (param != nullptr) param[i] = __float2bfloat16(p);
  }
}

__global__ void cast_f32_to_bf16_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst,
                                        long long n) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x)
    dst[i] = __float2bfloat16(src[i]);
}
__global__ void cast_bf16_to_f32_kernel(const __nv_bfloat16* __restrict__ src, float* __restrict__ dst,
                                        long long n) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x)
    dst[i] = __bfloat162float(src[i]);
}

}  // namespace axb

using namespace axb;

static inline int opt_grid(long long n) {
  long long b = (n + OPT_THREADS - 1) / OPT_THREADS;
  long long cap = (long long)sm_count() * 8;
  return (int)(b < 1 ? 1 : (b > cap ? cap : b));
}

extern "C" int axb_sumsq_partials(void) { return sm_count() * 8; }

// out[0] (+)= sum(g^2). scratch: axb_sumsq_partials() floats. grad_is_bf16 selects the dtype.
extern "C" int axb_sumsq(const void* g, long long n, int grad_is_bf16, float* scratch, float* out,
                         int accumulate, void* stream) {
  if (n <= 0) return AXB_LAUNCH_BAD_ARG;
  cudaStream_t s = (cudaStream_t)stream;
  const int grid = opt_grid(n);
  if (grad_is_bf16) sumsq_kernel<__nv_bfloat16><<<grid, OPT_THREADS, 0, s>>>((const __nv_bfloat16*)g, n, scratch);
  else sumsq_kernel<float><<<grid, OPT_THREADS, 0, s>>>((const float*)g, n, scratch);
  int rc = check_launch();
  if (rc) return rc;
  sumsq_final_kernel<<<1, 256, 0, s>>>(scratch, grid, out, accumulate);
  return check_launch();
}

extern "C" int axb_clip_coef(float* state, float max_norm, float skip_threshold, float grad_scale,
                             void* stream) {
  clip_coef_kernel<<<1, 1, 0, (cudaStream_t)stream>>>(state, max_norm, skip_threshold, grad_scale);
  return check_launch();
}

extern "C" int axb_adamw(float* master, void* param, const void* grad, int grad_is_bf16, float* m,
                         float* v, long long n, float lr, float beta1, float beta2, float eps, float wd,
                         float bc1, float bc2, const float* state, void* stream) {
  if (n <= 0) return AXB_LAUNCH_BAD_ARG;
  cudaStream_t s = (cudaStream_t)stream;
  const int grid = opt_grid(n);
  if (grad_is_bf16)
    adamw_kernel<__nv_bfloat16><<<grid, OPT_THREADS, 0, s>>>(master, (__nv_bfloat16*)param,
        (const __nv_bfloat16*)grad, m, v, n, lr, beta1, beta2, eps, wd, bc1, bc2, state);
  else
    adamw_kernel<float><<<grid, OPT_THREADS, 0, s>>>(master, (__nv_bfloat16*)param, (const float*)grad, m,
                                                    v, n, lr, beta1, beta2, eps, wd, bc1, bc2, state);
  return check_launch();
}

extern "C" int axb_cast_f32_bf16(const float* src, void* dst, long long n, void* stream) {
  if (n <= 0) return AXB_LAUNCH_BAD_ARG;
  cast_f32_to_bf16_kernel<<<opt_grid(n), 256, 0, (cudaStream_t)stream>>>(src, (__nv_bfloat16*)dst, n);
  return check_launch();
}
extern "C" int axb_cast_bf16_f32(const void* src, float* dst, long long n, void* stream) {
  if (n <= 0) return AXB_LAUNCH_BAD_ARG;
  cast_bf16_to_f32_kernel<<<opt_grid(n), 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)src, dst, n);
  return check_launch();
}
