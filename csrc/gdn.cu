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


// Backward of the recurrence, same decomposition (one CTA per 32 value columns of one (sequence, head)).
// The reverse sweep needs S_{t-1} and S_t at every token. They are not recovered by dividing by the decay (exp(g) can
// be tiny); instead the sequence is processed in chunks of GDN_CHUNK tokens from the back: the forward recurrence is
// replayed over a chunk from the state saved at its start (chunk-start states are produced by a first forward sweep),
// every intermediate state of the chunk is parked in a per-CTA scratch area in global memory, and the reverse sweep
// reads them back. With dS the gradient w.r.t. the state after token t:
//     dS   += scale * q_t do_t^T                    dq_t  = scale * S_t do_t
//     du    = dS^T k_t                              dk_t  = dS u_t + S'_t dr          (S'_t = a_t S_{t-1}, dr = -beta_t du)
//     dbeta = <du, v_t - r_t>                       dv_t  = beta_t du                 (r_t = S'_t^T k_t)
//     dS'   = dS + k_t dr^T                         dg_t  = a_t <dS', S_{t-1}>        dS <- a_t dS'
// dq, dk, dg and dbeta sum over ALL value columns: every CTA writes its 32-column partial into slice vb of
// [n_vblocks][T][H][...] buffers, which the caller adds up.
constexpr int GDN_CHUNK = 32;

template <int ROWS>
__global__ void __launch_bounds__(128)
gdn_bwd_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k, const __nv_bfloat16* __restrict__ v,
               const float* __restrict__ g, const float* __restrict__ beta, const int* __restrict__ cu_seqlens,
               const float* __restrict__ state_in, const __nv_bfloat16* __restrict__ d_o, const float* __restrict__ d_state_out,
               float* __restrict__ chunk_states,   // [n_seqs][H][n_vb][max_chunks][DK][32]
               float* __restrict__ scratch,        // [n_seqs][H][n_vb][GDN_CHUNK + 1][DK][32]
               float* __restrict__ dq_part, float* __restrict__ dk_part, float* __restrict__ dg_part, float* __restrict__ db_part,
               float* __restrict__ dv_out, float* __restrict__ d_state_in, int H, int dv, int T_total, int max_chunks, float scale) {
  constexpr int DK = ROWS * 4;
  const int j = threadIdx.x & 31, r = threadIdx.x >> 5;
  const int vb = blockIdx.x, h = blockIdx.y, sq = blockIdx.z, n_vb = gridDim.x;
  const int col = vb * GDN_BV + j;
  const bool col_ok = col < dv;
  const int t0 = cu_seqlens[sq], t1 = cu_seqlens[sq + 1];
  const int n_chunks = (t1 - t0 + GDN_CHUNK - 1) / GDN_CHUNK;
  __shared__ float sk[GDN_MAX_DK], sq_[GDN_MAX_DK];
  __shared__ float red[3][4][GDN_BV];
  __shared__ float srow[GDN_MAX_DK];           // per-row partial sums over the 32 columns (dq / dk)
  const long long cta = (static_cast<long long>(sq) * H + h) * n_vb + vb;
  float* cs = chunk_states + cta * max_chunks * DK * GDN_BV;
  float* sc = scratch + cta * (GDN_CHUNK + 1) * DK * GDN_BV;
  const long long sbase = ((static_cast<long long>(sq) * H + h) * DK) * dv;
  auto at = [&](float* base, int slot, int i) -> float& { return base[(static_cast<long long>(slot) * DK + (r * ROWS + i)) * GDN_BV + j]; };

  float S[ROWS];
  // ---- sweep 1: forward over the sequence, saving the state at the start of every chunk
#pragma unroll
  for (int i = 0; i < ROWS; ++i)
    S[i] = (state_in != nullptr && col_ok) ? state_in[sbase + static_cast<long long>(r * ROWS + i) * dv + col] : 0.f;
  for (int c = 0; c < n_chunks; ++c) {
#pragma unroll
    for (int i = 0; i < ROWS; ++i) at(cs, c, i) = S[i];
    const int e = min(t1, t0 + (c + 1) * GDN_CHUNK);
    for (int t = t0 + c * GDN_CHUNK; t < e; ++t) {
      const long long row = static_cast<long long>(t) * H + h;
      __syncthreads();
      for (int i = threadIdx.x; i < DK; i += 128) sk[i] = __bfloat162float(k[row * DK + i]);
      const float a = __expf(g[row]), b = beta[row];
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
#pragma unroll
      for (int i = 0; i < ROWS; ++i) S[i] += sk[r * ROWS + i] * u;
    }
  }
  // ---- sweep 2: chunks from the back
  float dS[ROWS];
#pragma unroll
  for (int i = 0; i < ROWS; ++i)
    dS[i] = (d_state_out != nullptr && col_ok) ? d_state_out[sbase + static_cast<long long>(r * ROWS + i) * dv + col] : 0.f;
  for (int c = n_chunks - 1; c >= 0; --c) {
    const int b0 = t0 + c * GDN_CHUNK, e = min(t1, b0 + GDN_CHUNK);
    // replay the chunk: slot n of the scratch holds the state BEFORE token b0 + n (slot e - b0: after the last one)
#pragma unroll
    for (int i = 0; i < ROWS; ++i) {
      S[i] = at(cs, c, i);
      at(sc, 0, i) = S[i];
    }
    for (int t = b0; t < e; ++t) {
      const long long row = static_cast<long long>(t) * H + h;
      __syncthreads();
      for (int i = threadIdx.x; i < DK; i += 128) sk[i] = __bfloat162float(k[row * DK + i]);
      const float a = __expf(g[row]), b = beta[row];
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
#pragma unroll
      for (int i = 0; i < ROWS; ++i) {
        S[i] += sk[r * ROWS + i] * u;
        at(sc, t - b0 + 1, i) = S[i];
      }
    }
    // reverse sweep over the chunk (each thread reads back exactly what it wrote: no fence needed)
    for (int t = e - 1; t >= b0; --t) {
      const long long row = static_cast<long long>(t) * H + h;
      __syncthreads();
      for (int i = threadIdx.x; i < DK; i += 128) {
        sk[i] = __bfloat162float(k[row * DK + i]);
        sq_[i] = __bfloat162float(q[row * DK + i]);
      }
      const float a = __expf(g[row]), b = beta[row];
      const float vt = col_ok ? __bfloat162float(v[row * dv + col]) : 0.f;
      const float dot_ = col_ok ? __bfloat162float(d_o[row * dv + col]) : 0.f;
      __syncthreads();
      float du = 0.f, rdot = 0.f;
#pragma unroll
      for (int i = 0; i < ROWS; ++i) {
        const float st = at(sc, t - b0 + 1, i);                 // S_t
        const float sp = a * at(sc, t - b0, i);                 // S'_t = a_t S_{t-1}
        dS[i] += scale * sq_[r * ROWS + i] * dot_;
        du += dS[i] * sk[r * ROWS + i];
        rdot += sp * sk[r * ROWS + i];
        S[i] = st;
      }
      red[0][r][j] = du;
      red[1][r][j] = rdot;
      __syncthreads();
      du = red[0][0][j] + red[0][1][j] + red[0][2][j] + red[0][3][j];
      const float rt = red[1][0][j] + red[1][1][j] + red[1][2][j] + red[1][3][j];
      const float u = b * (vt - rt);
      const float dr = -b * du;
      if (r == 0 && col_ok) dv_out[row * dv + col] = b * du;
      // column sums over the 32 lanes: dbeta, and per row dq / dk / the decay term
      float dbt = col_ok ? du * (vt - rt) : 0.f;
      float dgt = 0.f;
#pragma unroll
      for (int i = 0; i < ROWS; ++i) {
        const float sprev = at(sc, t - b0, i);
        const float sp = a * sprev;
        float dq_i = scale * S[i] * dot_;                        // S_t[i][j] do[j]
        float dk_i = dS[i] * u + sp * dr;
        const float dsp = dS[i] + sk[r * ROWS + i] * dr;         // dS'
        dgt += dsp * sprev;
        dS[i] = a * dsp;
        if (!col_ok) {
          dq_i = 0.f;
          dk_i = 0.f;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
          dq_i += __shfl_xor_sync(0xffffffffu, dq_i, o);
          dk_i += __shfl_xor_sync(0xffffffffu, dk_i, o);
        }
        if (j == 0) {
          const long long out = ((static_cast<long long>(vb) * T_total + t) * H + h) * DK + r * ROWS + i;
          dq_part[out] = dq_i;
          dk_part[out] = dk_i;
        }
      }
      dgt = col_ok ? dgt * a : 0.f;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        dgt += __shfl_xor_sync(0xffffffffu, dgt, o);
        dbt += __shfl_xor_sync(0xffffffffu, dbt, o);
      }
      if (j == 0) {
        red[2][r][0] = dgt;
        red[2][r][1] = dbt;
      }
      __syncthreads();
      if (threadIdx.x == 0) {
        const long long out = (static_cast<long long>(vb) * T_total + t) * H + h;
        dg_part[out] = red[2][0][0] + red[2][1][0] + red[2][2][0] + red[2][3][0];
        db_part[out] = red[2][0][1];          // every row group computed the same column sum of du (v - r)
      }
    }
  }
  if (d_state_in != nullptr && col_ok) {
#pragma unroll
    for (int i = 0; i < ROWS; ++i) d_state_in[sbase + static_cast<long long>(r * ROWS + i) * dv + col] = dS[i];
  }
  (void)srow;
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

// Backward. d_o: bf16 [T][H][dv]; d_state_out: fp32 [n_seqs][H][dk][dv] or null. Outputs: dv_out fp32 [T][H][dv];
// partials over the n_vb = ceil(dv / 32) value slices, to be summed over the leading dimension by the caller:
// dq_part, dk_part fp32 [n_vb][T][H][dk], dg_part, db_part fp32 [n_vb][T][H]; d_state_in fp32 like state_in or null.
// chunk_states: fp32 [n_seqs][H][n_vb][max_chunks][dk][32] with max_chunks >= ceil(longest sequence / 32);
// scratch: fp32 [n_seqs][H][n_vb][33][dk][32].
extern "C" int axb_gdn_bwd(const void* q, const void* k, const void* v, const float* g, const float* beta, const int* cu_seqlens,
                           int n_seqs, int H, int dk, int dv, int T_total, int max_chunks, float scale, const float* state_in,
                           const void* d_o, const float* d_state_out, float* chunk_states, float* scratch, float* dq_part,
                           float* dk_part, float* dg_part, float* db_part, float* dv_out, float* d_state_in, void* stream) {
  using namespace axb;
  if (n_seqs <= 0 || H <= 0 || dv <= 0 || max_chunks <= 0 || (dk != 64 && dk != 128 && dk != 256)) return AXB_LAUNCH_BAD_ARG;
  dim3 grid((dv + GDN_BV - 1) / GDN_BV, H, n_seqs);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  auto Q = static_cast<const __nv_bfloat16*>(q);
  auto K = static_cast<const __nv_bfloat16*>(k);
  auto V = static_cast<const __nv_bfloat16*>(v);
  auto DO = static_cast<const __nv_bfloat16*>(d_o);
#define AXB_GDN_BWD(R)                                                                                                  \
  gdn_bwd_kernel<R><<<grid, 128, 0, s>>>(Q, K, V, g, beta, cu_seqlens, state_in, DO, d_state_out, chunk_states, scratch, \
                                          dq_part, dk_part, dg_part, db_part, dv_out, d_state_in, H, dv, T_total, max_chunks, scale)
  if (dk == 64) AXB_GDN_BWD(16);
  else if (dk == 128) AXB_GDN_BWD(32);
  else AXB_GDN_BWD(64);
#undef AXB_GDN_BWD
  return check_launch();
}
