// Lightning-indexer backward (GLM-5 / DeepSeek-V3.2 sparse attention).
//
//   logits[s][j] = sum_h w[s][h] * relu(q[s][h] . k[j])
//
// Given g[s][t] = d loss / d logits[s][idx[s][t]] at the selected keys only:
//   dw[s][h]   = sum_t g * relu(q_h . k_t)
//   dq[s][h]   = sum_t g * w_h * [q_h . k_t > 0] * k_t
//   dk[idx t] += sum_h g * w_h * [q_h . k_t > 0] * q_h          (atomics: several queries select one key)
//
// One block per query, one warp per selected key at a time. A lane owns 4 of the 128 dims; the 32 partial
// dot products of a head group are summed with a transposing butterfly (31 shuffles instead of 160), after
// which lane h holds the dot product of head h. Every warp adds into its own copy of dq in shared memory,
// so no atomics are needed inside the block; the copies are summed at the end.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "host_utils.h"

namespace {

constexpr int IDX_D = 128;
constexpr int IDX_WARPS = 4;

__global__ void __launch_bounds__(IDX_WARPS * 32)
indexer_bwd_kernel(const float* __restrict__ g, const int* __restrict__ idx, const __nv_bfloat16* __restrict__ q,
                   const __nv_bfloat16* __restrict__ k, const float* __restrict__ w, float* __restrict__ dq,
                   float* __restrict__ dk, float* __restrict__ dw, int heads, int topk, int Skv, long long ldq,
                   long long ldk) {
  extern __shared__ float smem[];
  const int s = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float* q_s = smem;                                   // [heads][128]
  float* w_s = q_s + heads * IDX_D;                    // [heads]
  float* dw_s = w_s + heads;                           // [warps][heads]
  float* dq_s = dw_s + IDX_WARPS * heads;              // [warps][heads][128]
  const __nv_bfloat16* qrow = q + (long long)s * heads * ldq;
  for (int i = threadIdx.x; i < heads * IDX_D; i += blockDim.x)
    q_s[i] = __bfloat162float(qrow[(long long)(i / IDX_D) * ldq + (i % IDX_D)]);
  for (int i = threadIdx.x; i < heads; i += blockDim.x) w_s[i] = w[(long long)s * heads + i];
  for (int i = threadIdx.x; i < IDX_WARPS * heads; i += blockDim.x) dw_s[i] = 0.0f;
  for (int i = threadIdx.x; i < IDX_WARPS * heads * IDX_D; i += blockDim.x) dq_s[i] = 0.0f;
  __syncthreads();
  float* my_dq = dq_s + (long long)warp * heads * IDX_D;
  float* my_dw = dw_s + warp * heads;

  for (int t = warp; t < topk; t += IDX_WARPS) {
    const int j = idx[(long long)s * topk + t];
    const float gt = g[(long long)s * topk + t];
    if (j < 0 || j >= Skv || gt == 0.0f) continue;     // uniform over the warp
    const uint2 raw = *reinterpret_cast<const uint2*>(k + (long long)j * ldk + lane * 4);
    const __nv_bfloat162 k01 = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
    const __nv_bfloat162 k23 = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
    const float kv[4] = {__low2float(k01), __high2float(k01), __low2float(k23), __high2float(k23)};
    float dk_acc[4] = {0.f, 0.f, 0.f, 0.f};
    for (int h0 = 0; h0 < heads; h0 += 32) {
      float v[32];
#pragma unroll
      for (int h = 0; h < 32; ++h) {
        const float4 qv = *reinterpret_cast<const float4*>(q_s + (h0 + h) * IDX_D + lane * 4);
        v[h] = qv.x * kv[0] + qv.y * kv[1] + qv.z * kv[2] + qv.w * kv[3];
      }
#pragma unroll
      for (int off = 16; off >= 1; off >>= 1) {
        const bool upper = (lane & off) != 0;
#pragma unroll
        for (int i = 0; i < off; ++i) {
          const float send = upper ? v[i] : v[i + off];
          const float keep = upper ? v[i + off] : v[i];
          v[i] = keep + __shfl_xor_sync(0xffffffffu, send, off);
        }
      }
      const float dot = v[0];                          // head h0 + lane
      my_dw[h0 + lane] += gt * fmaxf(dot, 0.0f);
      const float coef = dot > 0.0f ? gt * w_s[h0 + lane] : 0.0f;
#pragma unroll 4
      for (int h = 0; h < 32; ++h) {
        const float c = __shfl_sync(0xffffffffu, coef, h);
        if (c != 0.0f) {                               // uniform over the warp
          float4* d = reinterpret_cast<float4*>(my_dq + (h0 + h) * IDX_D + lane * 4);
          float4 cur = *d;
          cur.x += c * kv[0];
          cur.y += c * kv[1];
          cur.z += c * kv[2];
          cur.w += c * kv[3];
          *d = cur;
          const float4 qv = *reinterpret_cast<const float4*>(q_s + (h0 + h) * IDX_D + lane * 4);
          dk_acc[0] += c * qv.x;
          dk_acc[1] += c * qv.y;
          dk_acc[2] += c * qv.z;
          dk_acc[3] += c * qv.w;
        }
      }
    }
    float* dkr = dk + (long long)j * IDX_D + lane * 4;
#pragma unroll
    for (int i = 0; i < 4; ++i) atomicAdd(dkr + i, dk_acc[i]);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < heads * IDX_D; i += blockDim.x) {
    float a = 0.0f;
#pragma unroll
    for (int wi = 0; wi < IDX_WARPS; ++wi) a += dq_s[(long long)wi * heads * IDX_D + i];
    dq[(long long)s * heads * IDX_D + i] = a;
  }
  for (int i = threadIdx.x; i < heads; i += blockDim.x) {
    float a = 0.0f;
#pragma unroll
    for (int wi = 0; wi < IDX_WARPS; ++wi) a += dw_s[wi * heads + i];
    dw[(long long)s * heads + i] = a;
  }
}


// ---------------------------------------------------------------------------------------------
// Row softmax over the selected keys for the dense-masked form of sparse latent attention.
// scores: fp32 [rows][ld] (raw q.k of one query chunk, rows = (query, head)); allowed: bytes [queries][n]
// (1 = the query selected this key). Writes p = exp(scale * score - lse) as bf16 (0 where not selected) and,
// unless ``lse_in`` is given (backward: reuse the forward's), the row's log-sum-exp. One block per row, two
// passes over the row (the second one hits L2); a row without any selected key gives zeros and lse = -inf.
__device__ __forceinline__ float block_reduce(float v, bool is_max, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
#pragma unroll
  for (int o = 16; o >= 1; o >>= 1) {
    const float u = __shfl_xor_sync(0xffffffffu, v, o);
    v = is_max ? fmaxf(v, u) : v + u;
  }
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  v = red[0];
  for (int i = 1; i < nw; ++i) v = is_max ? fmaxf(v, red[i]) : v + red[i];
  return v;
}

__global__ void __launch_bounds__(256)
masked_softmax_kernel(const float* __restrict__ scores, const unsigned char* __restrict__ allowed,
                      __nv_bfloat16* __restrict__ p, float* __restrict__ lse_out, const float* __restrict__ lse_in,
                      int heads, int n, long long ld, long long ldp, float scale) {
  __shared__ float red[8];
  const long long r = blockIdx.x;
  const float* row = scores + r * ld;
  const unsigned char* ok = allowed + (r / heads) * (long long)n;
  __nv_bfloat16* out = p + r * ldp;
  float lse;
  if (lse_in != nullptr) {
    lse = lse_in[r];
  } else {
    float m = -INFINITY;
    for (int j = threadIdx.x; j < n; j += blockDim.x)
      if (ok[j]) m = fmaxf(m, row[j] * scale);
    m = block_reduce(m, true, red);
    float sum = 0.0f;
    if (m > -INFINITY)
      for (int j = threadIdx.x; j < n; j += blockDim.x)
        if (ok[j]) sum += __expf(row[j] * scale - m);
    sum = block_reduce(sum, false, red);
    lse = (m > -INFINITY) ? m + __logf(sum) : -INFINITY;
    if (threadIdx.x == 0) lse_out[r] = lse;
  }
  const float base = (lse > -INFINITY) ? lse : 0.0f;
  for (int j = threadIdx.x; j < n; j += blockDim.x)
    out[j] = __float2bfloat16(ok[j] ? __expf(row[j] * scale - base) : 0.0f);
}

// ds = p * (dp - delta[row]) * scale as bf16 (p is already 0 outside the selection).
__global__ void __launch_bounds__(256)
softmax_bwd_kernel(const __nv_bfloat16* __restrict__ p, const float* __restrict__ dp, const float* __restrict__ delta,
                   __nv_bfloat16* __restrict__ ds, int n, long long ldp, long long lddp, float scale) {
  const long long r = blockIdx.x;
  const float d = delta[r];
  for (int j = threadIdx.x; j < n; j += blockDim.x)
    ds[r * ldp + j] = __float2bfloat16(__bfloat162float(p[r * ldp + j]) * (dp[r * lddp + j] - d) * scale);
}

}  // namespace

// g: fp32 [S][topk], idx: int32 [S][topk] (-1 = none), q: bf16 rows (s, h) with pitch ldq, k: bf16 [Skv][ldk],
// w: fp32 [S][heads]. Outputs fp32: dq [S][heads][128], dw [S][heads] (written), dk [Skv][128] (ADDED to: the
// caller zeroes it). heads % 32 == 0, head dim 128.
extern "C" int axb_indexer_bwd(const float* g, const int* idx, const void* q, const void* k, const float* w, float* dq,
                               float* dk, float* dw, int S, int heads, int topk, int Skv, int D, long long ldq,
                               long long ldk, void* stream) {
  using namespace axb;
  if (S <= 0 || topk <= 0 || Skv <= 0 || heads <= 0 || heads % 32 != 0 || heads > 64 || D != IDX_D || (ldk & 3))
    return AXB_LAUNCH_BAD_ARG;
  const size_t smem = sizeof(float) * ((size_t)heads * IDX_D + heads + IDX_WARPS * heads + (size_t)IDX_WARPS * heads * IDX_D);
  static size_t attr = 0;
  if (smem > attr) {
    if (cudaFuncSetAttribute(indexer_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
      return AXB_LAUNCH_CUDA_ERROR;
    attr = smem;
  }
  indexer_bwd_kernel<<<S, IDX_WARPS * 32, smem, static_cast<cudaStream_t>(stream)>>>(
      g, idx, static_cast<const __nv_bfloat16*>(q), static_cast<const __nv_bfloat16*>(k), w, dq, dk, dw, heads, topk, Skv,
      ldq, ldk);
  return check_launch();
}

extern "C" int axb_masked_softmax(const float* scores, const void* allowed, void* p, float* lse_out, const float* lse_in,
                                  long long rows, int heads, int n, long long ld, long long ldp, float scale, void* stream) {
  using namespace axb;
  if (rows <= 0 || rows > 0x7fffffffLL || heads <= 0 || n <= 0 || (lse_out == nullptr && lse_in == nullptr))
    return AXB_LAUNCH_BAD_ARG;
  masked_softmax_kernel<<<(unsigned)rows, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      scores, static_cast<const unsigned char*>(allowed), static_cast<__nv_bfloat16*>(p), lse_out, lse_in, heads, n, ld, ldp,
      scale);
  return check_launch();
}

extern "C" int axb_softmax_bwd(const void* p, const float* dp, const float* delta, void* ds, long long rows, int n,
                               long long ldp, long long lddp, float scale, void* stream) {
  using namespace axb;
  if (rows <= 0 || rows > 0x7fffffffLL || n <= 0) return AXB_LAUNCH_BAD_ARG;
  softmax_bwd_kernel<<<(unsigned)rows, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(p), dp, delta, static_cast<__nv_bfloat16*>(ds), n, ldp, lddp, scale);
  return check_launch();
}
