// Fused vocabulary head for PPO-style losses: per-token log-probability of the label and the
// entropy of softmax(hidden W^T / temperature), without ever materialising [T, V] logits.
//
//   forward   tcgen05 GEMM whose epilogue keeps, per row and per 128x256 tile, the running
//             (max, sum exp, sum z*exp) and the label's logit; a second small kernel merges the
//             per-tile partials into logprob[T], entropy[T], lse[T].
//   backward  the same GEMM recomputes the logits tile and its epilogue writes
//             dlogits = [g_lp (onehot - p) - g_ent p (z - lse + H)] / temperature   (bf16)
//             for a chunk of rows; dHidden and dW are then plain tcgen05 GEMMs over that chunk.
//
// Same contract as the reference's Triton ``linear_cross_entropy``
// (axon/utils/kernel/linear_cross_entropy.py:50-131, kernels.py:152-697).
#include "gemm_core.cuh"
#include "host_utils.h"

namespace axb {

struct StatsEpi {
  struct Params {
    float* partials;       // [M][num_n][3]  (max, sumexp, sum z*exp)
    float* label_logit;    // [M]
    const int* labels;     // [M], <0 = ignore
    int num_n;
    float inv_temp;
  };
  const Params& p;
  const GemmShape& sh;
  int row, n_blk;
  float m, s, sx;
  int label;
  __device__ StatsEpi(const Params& p_, int, int n_blk_, int row_, const GemmShape& sh_, int)
      : p(p_), sh(sh_), row(row_), n_blk(n_blk_), m(-INFINITY), s(0.f), sx(0.f) {
    label = row < sh.M ? p.labels[row] : -1;
  }
  __device__ __forceinline__ void chunk(int col0, const uint32_t (&acc)[32]) {
    if (row >= sh.M || col0 >= sh.N) return;
    float z[32];
    float cm = -INFINITY;
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      z[j] = (col0 + j < sh.N) ? __uint_as_float(acc[j]) * p.inv_temp : -INFINITY;
      cm = fmaxf(cm, z[j]);
    }
    if (label >= col0 && label < col0 + 32) {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (col0 + j == label) p.label_logit[row] = z[j];
    }
    const float nm = fmaxf(m, cm);
    const float a = __expf(m - nm);  // 0 on the first chunk (m = -inf)
    s *= a;
    sx *= a;
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      const float e = __expf(z[j] - nm);  // exp(-inf) = 0 for masked columns
      s += e;
      sx += (col0 + j < sh.N) ? z[j] * e : 0.f;
    }
    m = nm;
  }
  __device__ __forceinline__ void finish() {
    if (row >= sh.M) return;
    float* o = p.partials + ((long long)row * p.num_n + n_blk) * 3;
    o[0] = m;
    o[1] = s;
    o[2] = sx;
  }
};

// One warp per row merges the per-tile partials.
__global__ void lmhead_reduce_kernel(const float* __restrict__ partials, const float* __restrict__ label_logit,
                                     const int* __restrict__ labels, float* __restrict__ logprob,
                                     float* __restrict__ entropy, float* __restrict__ lse_out, int M,
                                     int num_n) {
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= M) return;
  float m = -INFINITY, s = 0.f, sx = 0.f;
  for (int i = lane; i < num_n; i += 32) {
    const float* o = partials + ((long long)row * num_n + i) * 3;
    const float pm = o[0], ps = o[1], px = o[2];
    const float nm = fmaxf(m, pm);
    const float a = (m == -INFINITY) ? 0.f : __expf(m - nm);
    const float b = (pm == -INFINITY) ? 0.f : __expf(pm - nm);
    s = s * a + ps * b;
    sx = sx * a + px * b;
    m = nm;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float pm = __shfl_xor_sync(0xffffffffu, m, o);
    const float ps = __shfl_xor_sync(0xffffffffu, s, o);
    const float px = __shfl_xor_sync(0xffffffffu, sx, o);
    const float nm = fmaxf(m, pm);
    const float a = (m == -INFINITY) ? 0.f : __expf(m - nm);
    const float b = (pm == -INFINITY) ? 0.f : __expf(pm - nm);
    s = s * a + ps * b;
    sx = sx * a + px * b;
    m = nm;
  }
  if (lane == 0) {
    const float lse = m + logf(s);
    lse_out[row] = lse;
    entropy[row] = lse - sx / s;
    logprob[row] = labels[row] >= 0 ? label_logit[row] - lse : 0.f;
  }
}

struct DLogitsEpi {
  struct Params {
    __nv_bfloat16* dlogits;  // [M][ld]
    long long ld;
    const int* labels;
    const float* lse;
    const float* entropy;
    const float* g_logprob;  // [M] or null (= 0)
    const float* g_entropy;  // [M] or null (= 0)
    float inv_temp;
  };
  const Params& p;
  const GemmShape& sh;
  int row, label;
  float lse, ent, glp, gent;
  __device__ DLogitsEpi(const Params& p_, int, int, int row_, const GemmShape& sh_, int)
      : p(p_), sh(sh_), row(row_) {
    const bool v = row < sh.M;
    label = v ? p.labels[row] : -1;
    lse = v ? p.lse[row] : 0.f;
    ent = v ? p.entropy[row] : 0.f;
    // label < 0: ignored token (no gradient) — except -2, which marks a valid token whose label lives in
    // another rank's vocabulary shard: it keeps the -g*p term and only drops the one-hot
    glp = (v && p.g_logprob && (label >= 0 || label == -2)) ? p.g_logprob[row] : 0.f;
    gent = (v && p.g_entropy) ? p.g_entropy[row] : 0.f;
  }
  __device__ __forceinline__ void chunk(int col0, const uint32_t (&acc)[32]) {
    if (row >= sh.M || col0 >= sh.N) return;
    float d[32];
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      const float z = __uint_as_float(acc[j]) * p.inv_temp;
      const float pr = __expf(z - lse);
      float g = -glp * pr - gent * pr * (z - lse + ent);
      if (col0 + j == label) g += glp;
      d[j] = g * p.inv_temp;
    }
    __nv_bfloat16* c = p.dlogits + (long long)row * p.ld + col0;
    if (col0 + 32 <= sh.N && (p.ld & 7) == 0) {
#pragma unroll
      for (int v = 0; v < 4; ++v) {
        uint4 o;
        o.x = pack_bf16x2(d[8 * v + 0], d[8 * v + 1]);
        o.y = pack_bf16x2(d[8 * v + 2], d[8 * v + 3]);
        o.z = pack_bf16x2(d[8 * v + 4], d[8 * v + 5]);
        o.w = pack_bf16x2(d[8 * v + 6], d[8 * v + 7]);
        reinterpret_cast<uint4*>(c)[v] = o;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (col0 + j < sh.N) c[j] = __float2bfloat16(d[j]);
    }
  }
  __device__ __forceinline__ void finish() {}
};

template <class Epi, class TM = DenseTiles>
static int launch_head(const void* hidden, const void* W, int M, int V, int H, long long ldh, long long ldw,
                       const typename Epi::Params& ep, int* status, cudaStream_t stream,
                       const typename TM::Params& tp = typename TM::Params{}) {
  CUtensorMap tmA, tmB;
  int rc = make_tmap_2d(&tmA, hidden, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, H, M, ldh * 2, GEMM_BK, GEMM_BM, true);
  if (rc) return rc;
  rc = make_tmap_2d(&tmB, W, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, H, V, ldw * 2, GEMM_BK, 256, true);
  if (rc) return rc;
  auto kern = gemm_tc_kernel<256, false, false, Epi, TM>;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, GemmSmem<256>::TOTAL) != cudaSuccess)
      return AXB_LAUNCH_CUDA_ERROR;
    attr_set = true;
  }
  const int tiles = ((M + GEMM_BM - 1) / GEMM_BM) * ((V + 255) / 256);
  int grid = sm_count();
  if (tiles < grid) grid = tiles;
  GemmShape sh{M, V, H, 1};
  kern<<<grid, GEMM_THREADS, GemmSmem<256>::TOTAL, stream>>>(tmA, tmB, sh, ep, status, tp);
  return check_launch();
}

// Vocabulary-parallel variant of the merge: one warp per row merges this rank's vocabulary tiles and
// stores (max, sum exp, sum z*exp, label logit or 0) as one float4 into slot [this rank][local row] of the
// statistics buffer of the rank that owns the row (peer store over NVLink; 16 bytes per token and rank).
struct PeerStats {
  float4* p[8];
};
__global__ void lmhead_reduce_to_peers_kernel(const float* __restrict__ partials, const float* __restrict__ label_logit,
                                              const int* __restrict__ labels_local, PeerStats stats, int rank,
                                              int rows_per_rank, int M, int num_n) {
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= M) return;
  float m = -INFINITY, s = 0.f, sx = 0.f;
  for (int i = lane; i < num_n; i += 32) {
    const float* o = partials + ((long long)row * num_n + i) * 3;
    const float pm = o[0], ps = o[1], px = o[2];
    const float nm = fmaxf(m, pm);
    const float a = (m == -INFINITY) ? 0.f : __expf(m - nm);
    const float b = (pm == -INFINITY) ? 0.f : __expf(pm - nm);
    s = s * a + ps * b;
    sx = sx * a + px * b;
    m = nm;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float pm = __shfl_xor_sync(0xffffffffu, m, o);
    const float ps = __shfl_xor_sync(0xffffffffu, s, o);
    const float px = __shfl_xor_sync(0xffffffffu, sx, o);
    const float nm = fmaxf(m, pm);
    const float a = (m == -INFINITY) ? 0.f : __expf(m - nm);
    const float b = (pm == -INFINITY) ? 0.f : __expf(pm - nm);
    s = s * a + ps * b;
    sx = sx * a + px * b;
    m = nm;
  }
  if (lane == 0) {
    const int owner = row / rows_per_rank, local = row - owner * rows_per_rank;
    const float lab = labels_local[row] >= 0 ? label_logit[row] : 0.f;
    stats.p[owner][(long long)rank * rows_per_rank + local] = make_float4(m, s, sx, lab);
  }
}

// After the barrier: merge the W slots of every local row in rank order (identical result on any schedule).
__global__ void lmhead_vp_finish_kernel(const float4* __restrict__ stats, const int* __restrict__ labels,
                                        float* __restrict__ logprob, float* __restrict__ entropy,
                                        float* __restrict__ lse_out, int world, int rows) {
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= rows) return;
  float m = -INFINITY;
  for (int w = 0; w < world; ++w) m = fmaxf(m, stats[(long long)w * rows + r].x);
  float s = 0.f, sx = 0.f, lab = 0.f;
  for (int w = 0; w < world; ++w) {
    const float4 v = stats[(long long)w * rows + r];
    const float sc = (v.x == -INFINITY) ? 0.f : __expf(v.x - m);
    s += v.y * sc;
    sx += v.z * sc;
    lab += v.w;
  }
  const float lse = m + logf(s);
  lse_out[r] = lse;
  entropy[r] = lse - sx / s;
  logprob[r] = labels[r] >= 0 ? lab - lse : 0.f;
}

}  // namespace axb

using namespace axb;

// Bytes of scratch the forward needs for M rows and vocabulary V.
extern "C" long long axb_lmhead_scratch_bytes(long long M, int V) {
  const long long num_n = (V + 255) / 256;
  return M * num_n * 3 * 4 + M * 4;
}

// logprob/entropy/lse: fp32 [M]. labels: int32 [M] (<0 ignored: logprob = 0).
extern "C" int axb_lmhead_fwd(const void* hidden, const void* W, const int* labels, float* logprob,
                              float* entropy, float* lse, int M, int V, int H, long long ldh, long long ldw,
                              float temperature, void* scratch, int* status, void* stream) {
  if (M <= 0 || V <= 0 || H <= 0 || (ldh & 7) || (ldw & 7) || temperature <= 0.f) return AXB_LAUNCH_BAD_ARG;
  cudaStream_t s = (cudaStream_t)stream;
  const int num_n = (V + 255) / 256;
  float* partials = reinterpret_cast<float*>(scratch);
  float* label_logit = partials + (long long)M * num_n * 3;
  StatsEpi::Params ep{partials, label_logit, labels, num_n, 1.f / temperature};
  int rc = launch_head<StatsEpi>(hidden, W, M, V, H, ldh, ldw, ep, status, s);
  if (rc) return rc;
  lmhead_reduce_kernel<<<(M + 7) / 8, 256, 0, s>>>(partials, label_logit, labels, logprob, entropy, lse, M, num_n);
  return check_launch();
}

// dlogits[M][ld] (bf16) from the saved lse/entropy and the upstream grads.
extern "C" int axb_lmhead_dlogits(const void* hidden, const void* W, const int* labels, const float* lse,
                                  const float* entropy, const float* g_logprob, const float* g_entropy,
                                  void* dlogits, long long ld, int M, int V, int H, long long ldh,
                                  long long ldw, float temperature, int* status, void* stream) {
  if (M <= 0 || V <= 0 || H <= 0 || (ldh & 7) || (ldw & 7) || temperature <= 0.f) return AXB_LAUNCH_BAD_ARG;
  DLogitsEpi::Params ep{(__nv_bfloat16*)dlogits, ld, labels, lse, entropy, g_logprob, g_entropy, 1.f / temperature};
  return launch_head<DLogitsEpi>(hidden, W, M, V, H, ldh, ldw, ep, status, (cudaStream_t)stream);
}


// Vocabulary-parallel forward, part 1. This rank holds W_shard [Vl][H] (vocabulary rows [v0, v0 + Vl)); the
// hidden states are row-sharded over the ranks (h_ptrs[r] = rank r's [rows_per_rank][H] shard in symmetric
// memory) and are read in place by the GEMM (all-gather fused, no gathered copy). labels_local: int32 [T],
// the label minus v0 where this shard owns it, otherwise negative. The per-token statistics go to the
// owners' buffers (stats_ptrs[r]: float4 [world][rows_per_rank]). scratch as for axb_lmhead_fwd(T, Vl).
extern "C" int axb_lmhead_vp_stats(const unsigned long long* h_ptrs, int world, int rank, const void* W_shard,
                                   const int* labels_local, int rows_per_rank, int Vl, int H, long long ldh,
                                   long long ldw, float temperature, void* scratch,
                                   const unsigned long long* stats_ptrs, int* status, void* stream) {
  if (world < 1 || world > 8 || rank < 0 || rank >= world || rows_per_rank <= 0 || rows_per_rank % GEMM_BM != 0 ||
      Vl <= 0 || (ldh & 7) || (ldw & 7) || temperature <= 0.f)
    return AXB_LAUNCH_BAD_ARG;
  cudaStream_t s = (cudaStream_t)stream;
  const int M = world * rows_per_rank;
  const int num_n = (Vl + 255) / 256;
  float* partials = reinterpret_cast<float*>(scratch);
  float* label_logit = partials + (long long)M * num_n * 3;
  StatsEpi::Params ep{partials, label_logit, labels_local, num_n, 1.f / temperature};
  PeerGatherTiles::Params tp;
  for (int r = 0; r < PeerGatherTiles::MAX_RANKS; ++r) {
    int rc = make_tmap_2d(&tp.maps[r], reinterpret_cast<const void*>(h_ptrs[r < world ? r : rank]),
                          CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, H, rows_per_rank, ldh * 2, GEMM_BK, GEMM_BM, true);
    if (rc) return rc;
  }
  tp.world = world;
  tp.rank = rank;
  tp.blocks_per_rank = rows_per_rank / GEMM_BM;
  int rc = launch_head<StatsEpi, PeerGatherTiles>(reinterpret_cast<const void*>(h_ptrs[rank]), W_shard, M, Vl, H, ldh, ldw,
                                                  ep, status, s, tp);
  if (rc) return rc;
  PeerStats st;
  for (int r = 0; r < 8; ++r) st.p[r] = reinterpret_cast<float4*>(stats_ptrs[r < world ? r : rank]);
  lmhead_reduce_to_peers_kernel<<<(M + 7) / 8, 256, 0, s>>>(partials, label_logit, labels_local, st, rank,
                                                           rows_per_rank, M, num_n);
  return check_launch();
}

// Part 2, after a device barrier: stats = this rank's buffer; labels = GLOBAL labels of the local rows.
extern "C" int axb_lmhead_vp_finish(const void* stats, const int* labels, float* logprob, float* entropy, float* lse,
                                    int world, int rows, void* stream) {
  if (world < 1 || rows <= 0) return AXB_LAUNCH_BAD_ARG;
  lmhead_vp_finish_kernel<<<(rows + 255) / 256, 256, 0, (cudaStream_t)stream>>>(
      reinterpret_cast<const float4*>(stats), labels, logprob, entropy, lse, world, rows);
  return check_launch();
}
