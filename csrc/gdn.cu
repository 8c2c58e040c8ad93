// Gated delta rule (Gated DeltaNet linear attention), recurrent form, forward.
//
// Per head a state S [dk x dv] evolves over the tokens of a sequence:
//     S   <- exp(g_t) * S
//     u_t  = beta_t * (v_t - S^T k_t)            (delta-rule correction of the value)
//     S   <- S + k_t u_t^T
//     o_t  = scale * S^T q_t
// (the recurrence behind ``chunk_gated_delta_rule`` / ``fused_recurrent_gated_delta_rule`` that the reference
// reaches through its GDN patch, axon/monkey_patches/transformers/qwen3_5_gdn.py). One CTA owns a 32-wide slice
// of the value dimension of one (sequence, head): 128 threads, thread (r, j) keeps rows r*dk/4 .. of column j
// of S in registers, k_t / q_t are staged in shared memory, the two dk-long dot products per token are
// reduced over the four row groups through shared memory. The sequence is walked token by token, so the
// kernel is latency bound (about a microsecond per token and CTA) and meant for decode-length steps, state
// carry-over and as the oracle-checked baseline of a chunked tensor-core version.
#include "ptx.cuh"
#include "host_utils.h"

namespace axb {

constexpr int GDN_BV = 32;
constexpr int GDN_MAX_DK = 256;

template <int ROWS>   // rows of S per thread = dk / 4
__global__ void __launch_bounds__(128)
gdn_fwd_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k, const __nv_bfloat16* __restrict__ v,
               const float* __restrict__ g, const float* __restrict__ beta, const int* __restrict__ cu_seqlens,
               const float* __restrict__ state_in, float* __restrict__ state_out, __nv_bfloat16* __restrict__ o, int H,
               int dv, float scale) {
  constexpr int DK = ROWS * 4;
  const int j = threadIdx.x & 31, r = threadIdx.x >> 5;
  const int vb = blockIdx.x, h = blockIdx.y, sq = blockIdx.z;
  const int col = vb * GDN_BV + j;
  const bool col_ok = col < dv;
  const int t0 = cu_seqlens[sq], t1 = cu_seqlens[sq + 1];
  __shared__ float sk[GDN_MAX_DK], sq_[GDN_MAX_DK];
  __shared__ float red[2][4][GDN_BV];
  float S[ROWS];
  const long long sbase = ((static_cast<long long>(sq) * H + h) * DK) * dv;
#pragma unroll
  for (int i = 0; i < ROWS; ++i)
    S[i] = (state_in != nullptr && col_ok) ? state_in[sbase + static_cast<long long>(r * ROWS + i) * dv + col] : 0.f;
  for (int t = t0; t < t1; ++t) {
    const long long row = static_cast<long long>(t) * H + h;
    for (int i = threadIdx.x; i < DK; i += 128) {
      sk[i] = __bfloat162float(k[row * DK + i]);
      sq_[i] = __bfloat162float(q[row * DK + i]);
    }
    const float a = __expf(g[row]);
    const float b = beta[row];
    const float vt = col_ok ? __bfloat162float(v[row * dv + col]) : 0.f;
    __syncthreads();
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < ROWS; ++i) {
      S[i] *= a;
      dot += S[i] * sk[r * ROWS + i];
    }
    red[0][r][j] = dot;
    __syncthreads();
    const float u = b * (vt - (red[0][0][j] + red[0][1][j] + red[0][2][j] + red[0][3][j]));
    float od = 0.f;
#pragma unroll
    for (int i = 0; i < ROWS; ++i) {
      S[i] += sk[r * ROWS + i] * u;
      od += S[i] * sq_[r * ROWS + i];
    }
    red[1][r][j] = od;
    __syncthreads();
    if (r == 0 && col_ok)
      o[row * dv + col] = __float2bfloat16(scale * (red[1][0][j] + red[1][1][j] + red[1][2][j] + red[1][3][j]));
  }
  if (state_out != nullptr && col_ok) {
#pragma unroll
    for (int i = 0; i < ROWS; ++i) state_out[sbase + static_cast<long long>(r * ROWS + i) * dv + col] = S[i];
  }
}

}  // namespace axb

// q, k: bf16 [T][H][dk]; v, o: bf16 [T][H][dv]; g (log decay), beta: fp32 [T][H]; cu_seqlens: int32 [n_seqs + 1];
// state_in / state_out: fp32 [n_seqs][H][dk][dv] or null. dk in {64, 128, 256}.
extern "C" int axb_gdn_fwd(const void* q, const void* k, const void* v, const float* g, const float* beta,
                           const int* cu_seqlens, int n_seqs, int H, int dk, int dv, float scale, const float* state_in,
                           float* state_out, void* o, void* stream) {
  using namespace axb;
  if (n_seqs <= 0 || H <= 0 || dv <= 0 || (dk != 64 && dk != 128 && dk != 256)) return AXB_LAUNCH_BAD_ARG;
  dim3 grid((dv + GDN_BV - 1) / GDN_BV, H, n_seqs);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  auto Q = static_cast<const __nv_bfloat16*>(q);
  auto K = static_cast<const __nv_bfloat16*>(k);
  auto V = static_cast<const __nv_bfloat16*>(v);
  auto O = static_cast<__nv_bfloat16*>(o);
  if (dk == 64) gdn_fwd_kernel<16><<<grid, 128, 0, s>>>(Q, K, V, g, beta, cu_seqlens, state_in, state_out, O, H, dv, scale);
  else if (dk == 128) gdn_fwd_kernel<32><<<grid, 128, 0, s>>>(Q, K, V, g, beta, cu_seqlens, state_in, state_out, O, H, dv, scale);
  else gdn_fwd_kernel<64><<<grid, 128, 0, s>>>(Q, K, V, g, beta, cu_seqlens, state_in, state_out, O, H, dv, scale);
  return check_launch();
}
