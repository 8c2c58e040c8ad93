// Weight-streaming GEMM for token batches of a few to a few hundred rows (the decode step):
//
//   out[tokens][feats] = X[tokens][K] * W[feats][K]^T          bf16 in, fp32 accumulate, bf16 / fp32 out
//
// Such a product is bound by reading W once from HBM, so the kernel is laid out around the weight
// stream rather than around the tensor core:
//   * weights ride on the 128-row side of tcgen05.mma ("swap-AB"), the tokens are the MMA's N dimension,
//     which is a RUN-TIME value here (any multiple of 16 up to 256): the instruction descriptor, the
//     TMA box of X, the stage size and the number of pipeline stages all follow the padded token count,
//     so a batch of 48 tokens moves 48 rows of activations per K block, not 256;
//   * one CTA per (128-feature tile, token tile, K split); shared memory is sized so that two CTAs fit
//     on an SM, which keeps > 10 MB of weight bytes in flight across the GPU (what 6.5 TB/s times the
//     loaded memory latency asks for) without a persistent scheduler;
//   * K is split when the product has too few tiles to cover the SMs. Partial tiles go to an fp32
//     workspace that stays in L2, the CTA that arrives LAST at the tile's counter sums the partials in
//     split order (so the result does not depend on which CTA that was) and writes the output. Nobody
//     waits for anybody: there is no spin, no cluster constraint and no second launch. The counter is
//     reset by the CTA that consumed it, so a captured graph can replay the launch.
//
// Warps: 0 = TMA producer, 1 = MMA issuer + TMEM owner, 2-5 = epilogue (TMEM lane quarters).
// Every mbarrier wait is bounded; on a timeout the CTA records an error in the status word, still
// takes part in the counter protocol and frees its TMEM.
#include "gemm_core.cuh"
#include "host_utils.h"

namespace axb {

#ifdef AXB_TIMELINE
// Development aid (compiled only with -DAXB_TIMELINE): per-CTA timestamps of the kernel's phases.
__device__ unsigned long long* g_stream_timeline = nullptr;
__device__ __forceinline__ void stl_mark(int slot) {
  if (g_stream_timeline != nullptr) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    g_stream_timeline[((blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x) * 8 + slot] = t;
  }
}
#define AXB_STL(slot, cond) do { if (cond) stl_mark(slot); } while (0)
#else
#define AXB_STL(slot, cond) do { } while (0)
#endif

constexpr int STREAM_W_BYTES = GEMM_BM * GEMM_BK * 2;   // 16 KB of weights per stage
constexpr int STREAM_MAX_STAGES = 12;
constexpr int STREAM_BAR_BYTES = 256;

__device__ __forceinline__ void epi_bar_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

__global__ void __launch_bounds__(GEMM_THREADS)
gemm_stream_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX, int feats,
                   int tokens, int K, int bn, int stages, int tmem_cols, float* __restrict__ ws,
                   unsigned int* __restrict__ counters, void* __restrict__ out, long long ldc, int out_fp32,
                   int* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  const int stage_bytes = STREAM_W_BYTES + bn * (GEMM_BK * 2);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + stages * stage_bytes);
  uint64_t* full = bars;
  uint64_t* empty = bars + STREAM_MAX_STAGES;
  uint64_t* acc_full = bars + 2 * STREAM_MAX_STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_full + 1);
  volatile uint32_t* arrival = tmem_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  AXB_STL(0, threadIdx.x == 0);
  const int split = blockIdx.x;
  const int S = gridDim.x;
  const int m_blk = blockIdx.y;
  const int n_blk = blockIdx.z;
  const int tile_id = n_blk * gridDim.y + m_blk;
  const int num_k = (K + GEMM_BK - 1) / GEMM_BK;
  const int k_per = (num_k + S - 1) / S;
  const int kb0 = split * k_per;
  const int kb1 = min(num_k, kb0 + k_per);

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(acc_full, 1);
    mbar_fence_init();
    tma_prefetch_desc(&tmW);
    tma_prefetch_desc(&tmX);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, static_cast<uint32_t>(tmem_cols));
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  AXB_STL(1, threadIdx.x == 0);

  if (warp == 0) {
    if (lane == 0) {
      int s = 0;
      uint32_t ph = 0;
      for (int kb = kb0; kb < kb1; ++kb) {
        if (!mbar_wait(&empty[s], ph ^ 1)) {
          report_error(status, AXB_ERR_WAIT_EMPTY);
          break;
        }
        uint8_t* sW = smem + s * stage_bytes;
        mbar_expect_tx(&full[s], static_cast<uint32_t>(stage_bytes));
        tma_load_2d(sW, &tmW, &full[s], kb * GEMM_BK, m_blk * GEMM_BM);
        tma_load_2d(sW + STREAM_W_BYTES, &tmX, &full[s], kb * GEMM_BK, n_blk * bn);
        if (++s == stages) {
          s = 0;
          ph ^= 1;
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = umma_idesc(GEMM_BM, static_cast<uint32_t>(bn), 0u, 0u);
      int s = 0;
      uint32_t ph = 0;
      bool issued = kb0 < kb1;
      for (int kb = kb0; kb < kb1; ++kb) {
        if (!mbar_wait(&full[s], ph)) {
          report_error(status, AXB_ERR_WAIT_FULL);
          issued = false;
          break;
        }
        tc_fence_after();
        AXB_STL(2, kb == kb0);
        const uint32_t a0 = smem_u32(smem + s * stage_bytes);
        const uint32_t b0 = a0 + STREAM_W_BYTES;
#pragma unroll
        for (int j = 0; j < GEMM_BK / 16; ++j)
          umma_f16_ss(tmem_base, umma_smem_desc(a0 + j * 32, 16, 1024), umma_smem_desc(b0 + j * 32, 16, 1024),
                      idesc, (kb != kb0 || j != 0) ? 1u : 0u);
        tc_commit(&empty[s]);
        if (++s == stages) {
          s = 0;
          ph ^= 1;
        }
      }
      if (issued) tc_commit(acc_full);
      AXB_STL(3, true);
    }
  } else {
    // ---------------------------------------------------------------- epilogue (128 threads)
    bool ok = kb0 < kb1;
    if (ok && !mbar_wait(acc_full, 0)) {
      report_error(status, AXB_ERR_WAIT_TMEM_FULL);
      ok = false;
    }
    tc_fence_after();
    AXB_STL(4, threadIdx.x == 64);
    const int q = warp & 3;
    const int row = q * 32 + lane;                 // feature row inside the tile = TMEM lane
    const int f = m_blk * GEMM_BM + row;
    const int tok0 = n_blk * bn;
    const int jmax = min(bn, tokens - tok0);       // real tokens of this tile
    const uint32_t t0 = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
    if (S == 1) {
      if (ok) {
#pragma unroll 1
        for (int c0 = 0; c0 < jmax; c0 += 16) {
          uint32_t acc[16];
          tmem_ld_32x16(t0 + c0, acc);
          tmem_ld_wait();
          if (f < feats) {
            if (out_fp32) {
              float* o = reinterpret_cast<float*>(out) + static_cast<long long>(tok0 + c0) * ldc + f;
#pragma unroll
              for (int j = 0; j < 16; ++j)
                if (c0 + j < jmax) o[static_cast<long long>(j) * ldc] = __uint_as_float(acc[j]);
            } else {
              __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(out) + static_cast<long long>(tok0 + c0) * ldc + f;
#pragma unroll
              for (int j = 0; j < 16; ++j)
                if (c0 + j < jmax) o[static_cast<long long>(j) * ldc] = __float2bfloat16(__uint_as_float(acc[j]));
            }
          }
        }
      }
    } else {
      // partial tile -> workspace [tile][split][token j][128 feature rows] (a warp writes 128 contiguous bytes)
      float* my = ws + (static_cast<long long>(tile_id) * S + split) * bn * GEMM_BM;
      if (ok) {
#pragma unroll 1
        for (int c0 = 0; c0 < jmax; c0 += 16) {
          uint32_t acc[16];
          tmem_ld_32x16(t0 + c0, acc);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 16; ++j)
            if (c0 + j < jmax) __stcg(my + (c0 + j) * GEMM_BM + row, __uint_as_float(acc[j]));
        }
      }
      __threadfence();
      epi_bar_sync();
      const int e = threadIdx.x - 64;
      if (e == 0) *arrival = atomicAdd(&counters[tile_id], 1u);
      epi_bar_sync();
      AXB_STL(5, threadIdx.x == 64);
      if (*arrival == static_cast<uint32_t>(S - 1)) {
        // last CTA of this tile: sum the S partials in split order, 4 features x 1 token per thread and step
        __threadfence();
        const int l4 = (e & 31) * 4;               // first of this thread's 4 feature rows
        const int f4 = m_blk * GEMM_BM + l4;
        const float* base = ws + static_cast<long long>(tile_id) * S * bn * GEMM_BM + l4;
        const long long sstride = static_cast<long long>(bn) * GEMM_BM;
#pragma unroll 1
        for (int j0 = (e >> 5); j0 < jmax; j0 += 16) {
          float4 sum[4];
#pragma unroll
          for (int u = 0; u < 4; ++u) sum[u] = make_float4(0.f, 0.f, 0.f, 0.f);
          for (int s = 0; s < S; ++s) {
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              const int j = j0 + 4 * u;
              if (j < jmax) {
                const float4 v = __ldcg(reinterpret_cast<const float4*>(base + s * sstride + j * GEMM_BM));
                sum[u].x += v.x;
                sum[u].y += v.y;
                sum[u].z += v.z;
                sum[u].w += v.w;
              }
            }
          }
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int j = j0 + 4 * u;
            if (j < jmax && f4 < feats) {   // feats is a multiple of 4 (checked on the host)
              if (out_fp32) {
                *reinterpret_cast<float4*>(reinterpret_cast<float*>(out) + static_cast<long long>(tok0 + j) * ldc + f4) = sum[u];
              } else {
                uint2 p;
                p.x = pack_bf16x2(sum[u].x, sum[u].y);
                p.y = pack_bf16x2(sum[u].z, sum[u].w);
                *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(out) + static_cast<long long>(tok0 + j) * ldc + f4) = p;
              }
            }
          }
        }
        if (e == 0) counters[tile_id] = 0u;        // ready for the next launch (graph replay)
        AXB_STL(6, threadIdx.x == 64);
      }
    }
    tc_fence_before();
  }

  __syncthreads();
  AXB_STL(7, threadIdx.x == 0);
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, static_cast<uint32_t>(tmem_cols));
  }
}

struct StreamPlan {
  int bn, tok_tiles, feat_tiles, splits, stages, tmem_cols;
  long long ws_floats;
  int smem_bytes;
};

static int g_force_splits = 0;        // tuning hooks (0 = heuristic)
static int g_max_bn = 128;
static int g_smem_budget = 108 * 1024;
static int g_reduce_kb = 256;
static int g_min_kblocks = 8;
static int g_target_ctas = 0;         // 0: two per SM

static StreamPlan make_plan(int tokens, int feats, int K) {
  StreamPlan p;
  const int max_bn = g_max_bn < 16 ? 16 : (g_max_bn > 256 ? 256 : g_max_bn / 16 * 16);
  p.tok_tiles = (tokens + max_bn - 1) / max_bn;
  const int per = (tokens + p.tok_tiles - 1) / p.tok_tiles;
  p.bn = (per + 15) / 16 * 16;
  p.feat_tiles = (feats + GEMM_BM - 1) / GEMM_BM;
  const int tiles = p.tok_tiles * p.feat_tiles;
  const int stage_bytes = STREAM_W_BYTES + p.bn * GEMM_BK * 2;
  int st = g_smem_budget / stage_bytes;
  p.stages = st < 2 ? 2 : (st > STREAM_MAX_STAGES ? STREAM_MAX_STAGES : st);
  p.smem_bytes = p.stages * stage_bytes + STREAM_BAR_BYTES + 1024;
  const int num_k = (K + GEMM_BK - 1) / GEMM_BK;
  const int target = g_target_ctas > 0 ? g_target_ctas : 2 * sm_count();
  int s = target / tiles;
  if (s < 1) s = 1;
  const int by_k = num_k / g_min_kblocks;                    // at least this many K blocks per CTA
  if (s > by_k) s = by_k;
  const int by_reduce = g_reduce_kb * 1024 / (p.bn * GEMM_BM * 4);   // what the last CTA has to read back
  if (s > by_reduce) s = by_reduce;
  if (s > 16) s = 16;
  if (g_force_splits > 0) s = g_force_splits;
  if (s < 1) s = 1;
  while (s > 1 && (s - 1) * ((num_k + s - 1) / s) >= num_k) --s;   // every split owns at least one K block
  p.splits = s;
  int c = 32;
  while (c < p.bn) c *= 2;
  p.tmem_cols = c;
  p.ws_floats = s > 1 ? static_cast<long long>(tiles) * s * p.bn * GEMM_BM : 0;
  return p;
}

}  // namespace axb

#ifdef AXB_TIMELINE
extern "C" int axb_gemm_stream_set_timeline(unsigned long long* buf) {
  return cudaMemcpyToSymbol(axb::g_stream_timeline, &buf, sizeof(buf)) == cudaSuccess ? 0 : -4;
}
#endif

// Tuning hooks for experiments; a value of 0 (or less) keeps the current setting of that knob.
extern "C" void axb_gemm_stream_tune(int force_splits, int max_bn, int smem_budget_kb, int reduce_kb,
                                     int min_kblocks, int target_ctas) {
  using namespace axb;
  g_force_splits = force_splits < 0 ? 0 : force_splits;
  if (max_bn > 0) g_max_bn = max_bn;
  if (smem_budget_kb > 0) g_smem_budget = smem_budget_kb * 1024;
  if (reduce_kb > 0) g_reduce_kb = reduce_kb;
  if (min_kblocks > 0) g_min_kblocks = min_kblocks;
  g_target_ctas = target_ctas < 0 ? 0 : target_ctas;
}

// Workspace the launch of this shape needs: fp32 elements of partial tiles (0 without a K split) and the
// number of per-tile arrival counters (zero-initialised once by the caller, self-resetting afterwards).
extern "C" int axb_gemm_stream_workspace(int tokens, int feats, int K, long long* ws_floats, int* n_counters,
                                         int* splits, int* bn) {
  using namespace axb;
  if (tokens <= 0 || feats <= 0 || K <= 0) return AXB_LAUNCH_BAD_ARG;
  const StreamPlan p = make_plan(tokens, feats, K);
  if (ws_floats) *ws_floats = p.ws_floats;
  if (n_counters) *n_counters = p.tok_tiles * p.feat_tiles;
  if (splits) *splits = p.splits;
  if (bn) *bn = p.bn;
  return AXB_LAUNCH_OK;
}

// out[tokens][ldc] = X[tokens][ldx] * W[feats][ldw]^T. `ws` / `counters` as sized by
// axb_gemm_stream_workspace for the same shape (and the same tuning state).
extern "C" int axb_gemm_stream(const void* X, const void* W, void* out, int tokens, int feats, int K, long long ldx,
                               long long ldw, long long ldc, int out_fp32, float* ws, unsigned int* counters,
                               int* status, void* stream) {
  using namespace axb;
  if (tokens <= 0 || feats <= 0 || K <= 0 || (ldx & 7) || (ldw & 7) || (feats & 3) || (ldc & 3)) return AXB_LAUNCH_BAD_ARG;
  const StreamPlan p = make_plan(tokens, feats, K);
  if (p.splits > 1 && (ws == nullptr || counters == nullptr)) return AXB_LAUNCH_BAD_ARG;
  if (p.tok_tiles > 65535 || p.feat_tiles > 65535) return AXB_LAUNCH_TOO_LARGE;
  CUtensorMap tmW, tmX;
  int rc = make_tmap_2d(&tmW, W, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, feats, ldw * 2, GEMM_BK, GEMM_BM, true);
  if (rc != AXB_LAUNCH_OK) return rc;
  rc = make_tmap_2d(&tmX, X, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, tokens, ldx * 2, GEMM_BK, p.bn, true);
  if (rc != AXB_LAUNCH_OK) return rc;
  static int smem_set = 0;
  if (p.smem_bytes > smem_set) {
    if (cudaFuncSetAttribute(gemm_stream_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, p.smem_bytes) != cudaSuccess)
      return AXB_LAUNCH_CUDA_ERROR;
    smem_set = p.smem_bytes;
  }
  dim3 grid(p.splits, p.feat_tiles, p.tok_tiles);
  gemm_stream_kernel<<<grid, GEMM_THREADS, p.smem_bytes, static_cast<cudaStream_t>(stream)>>>(
      tmW, tmX, feats, tokens, K, p.bn, p.stages, p.tmem_cols, ws, counters, out, ldc, out_fp32, status);
  return check_launch();
}
