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
    glp = (v && p.g_logprob && label >= 0) ? p.g_logprob[row] : 0.f;
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

template <class Epi>
static int launch_head(const void* hidden, const void* W, int M, int V, int H, long long ldh, long long ldw,
                       const typename Epi::Params& ep, int* status, cudaStream_t stream) {
  CUtensorMap tmA, tmB;
  int rc = make_tmap_2d(&tmA, hidden, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, H, M, ldh * 2, GEMM_BK, GEMM_BM, true);
  if (rc) return rc;
  rc = make_tmap_2d(&tmB, W, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, H, V, ldw * 2, GEMM_BK, 256, true);
  if (rc) return rc;
  auto kern = gemm_tc_kernel<256, false, false, Epi>;
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
  kern<<<grid, GEMM_THREADS, GemmSmem<256>::TOTAL, stream>>>(tmA, tmB, sh, ep, status, DenseTiles::Params{});
  return check_launch();
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
