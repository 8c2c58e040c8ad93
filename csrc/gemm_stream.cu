// Weight-streaming GEMM for token batches of a few to a few hundred rows (the decode step):
//
//   out[tokens][feats] = X[tokens][K] * W[feats][K]^T          bf16 in, fp32 accumulate, bf16 / fp32 out
//
// Such a product is bound by reading W once from HBM, so the kernel is laid out around the weight
// stream rather than around the tensor core:
//   * weights ride on the 128-row side of tcgen05.mma ("swap-AB"), the tokens are the MMA's N dimension,
//     which is a RUN-TIME value here (any multiple of 16 up to 256): the instruction descriptor, the
//     TMA box of X and the ring sizes all follow the padded token count, so a batch of 48 tokens moves
//     48 rows of activations per K block, not 256;
//   * W and X travel through SEPARATE shared-memory rings. X tiles are L2 hits with a short latency and
//     get a shallow ring; everything else is a deep ring of 16 KB weight tiles, because under load HBM
//     answers after a few microseconds and ~160 KB of weight bytes per SM must be in flight to keep
//     6.5 TB/s busy. The W producer starts at once; only the X producer waits for the previous kernel
//     of the stream (programmatic dependent launch), so the weight stream of this product overlaps the
//     tail of whatever produced its activations;
//   * one CTA per (128-feature tile, token tile, K split), two CTAs per SM (a one-CTA-per-SM plan with
//     rings twice as deep exists behind a knob; it measured slower);
//   * K is split when the product has too few tiles to cover the SMs. The splits of a tile draw a
//     ticket when their accumulator is complete. All but the last add their partial tile into one fp32
//     accumulation tile (bulk reductions executed by the L2) and count themselves done; the CTA with
//     the last ticket keeps its partial in TMEM, waits (bounded) for the others - which are by then in
//     their own epilogues, never still to be scheduled -, pulls the accumulation tile into shared
//     memory, adds its own part, writes the output and stores zeros back, so tile and counters are
//     ready for the next launch (graph replay). The order of the fp32 additions is not fixed for more
//     than two splits; a bit-reproducible variant (partials side by side, summed in split order by
//     the last CTA) is kept behind a switch.
//
// Warps: 0 = W producer, 1 = MMA issuer + TMEM owner, 2-5 = epilogue (TMEM lane quarters), 6 = X
// producer. Every wait is bounded; on a timeout the CTA records an error in the status word, still
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

constexpr int STREAM_THREADS = 224;
constexpr int STREAM_W_BYTES = GEMM_BM * GEMM_BK * 2;   // 16 KB of weights per W stage
constexpr int STREAM_MAX_W = 16;
constexpr int STREAM_MAX_X = 8;
constexpr int STREAM_BAR_BYTES = 512;

__device__ __forceinline__ void epi_bar_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

__device__ __forceinline__ unsigned int ld_acquire_u32(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// out rows [tok_first, +out_rows) of this tile from the fp32 staging area [row j][128 features]; with `zero`
// all `rows` rows of the area are cleared on the way (it is stored back as the next launch's empty accumulation tile).
__device__ __forceinline__ void stage_to_out(float* stg, int rows, int out_rows, int e, void* out, long long ldc,
                                             int out_fp32, int tok_first, int f4, int feats, bool zero) {
  const int l4 = (e & 31) * 4;
#pragma unroll 2
  for (int j = (e >> 5); j < rows; j += 4) {
    float4* sp = reinterpret_cast<float4*>(stg + j * GEMM_BM + l4);
    const float4 v = *sp;
    if (zero) *sp = make_float4(0.f, 0.f, 0.f, 0.f);
    if (j < out_rows && f4 < feats) {   // rows past out_rows are token padding; feats is a multiple of 4 (checked on the host)
      if (out_fp32) {
        *reinterpret_cast<float4*>(reinterpret_cast<float*>(out) + static_cast<long long>(tok_first + j) * ldc + f4) = v;
      } else {
        uint2 p;
        p.x = pack_bf16x2(v.x, v.y);
        p.y = pack_bf16x2(v.z, v.w);
        *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(out) + static_cast<long long>(tok_first + j) * ldc + f4) = p;
      }
    }
  }
}

// TMEM accumulator columns [r0, r0 + rows) of this thread's feature row -> staging area (set or add).
template <bool ADD>
__device__ __forceinline__ void tmem_to_stage(uint32_t t0, float* stg, int r0, int rows, int row) {
#pragma unroll 1
  for (int c0 = r0; c0 < r0 + rows; c0 += 16) {
    uint32_t acc[16];
    tmem_ld_32x16(t0 + c0, acc);
    tmem_ld_wait();
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      float* p = stg + (c0 - r0 + j) * GEMM_BM + row;
      if (ADD) *p += __uint_as_float(acc[j]);
      else *p = __uint_as_float(acc[j]);
    }
  }
}

__global__ void __launch_bounds__(STREAM_THREADS)
gemm_stream_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX, int feats,
                   int tokens, int K, int bn, int dw, int dx, int tmem_cols, float* __restrict__ ws,
                   unsigned int* __restrict__ counters, void* __restrict__ out, long long ldc, int out_fp32,
                   int accumulate_mode, int* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  const int xbytes = bn * (GEMM_BK * 2);
  uint8_t* smemX = smem + dw * STREAM_W_BYTES;
  const int ring_bytes = dw * STREAM_W_BYTES + dx * xbytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + ring_bytes);
  uint64_t* fullW = bars;
  uint64_t* emptyW = fullW + STREAM_MAX_W;
  uint64_t* fullX = emptyW + STREAM_MAX_W;
  uint64_t* emptyX = fullX + STREAM_MAX_X;
  uint64_t* acc_full = emptyX + STREAM_MAX_X;
  uint64_t* red_full = acc_full + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(red_full + 1);
  volatile uint32_t* ticket_slot = tmem_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  AXB_STL(0, threadIdx.x == 0);
  grid_launch_dependents();      // the next kernel of the stream may start its own prologue / weight prefetch
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
    for (int s = 0; s < dw; ++s) {
      mbar_init(&fullW[s], 1);
      mbar_init(&emptyW[s], 1);
    }
    for (int s = 0; s < dx; ++s) {
      mbar_init(&fullX[s], 1);
      mbar_init(&emptyX[s], 1);
    }
    mbar_init(acc_full, 1);
    mbar_init(red_full, 1);
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
    if (lane == 0) {   // weights: independent of the previous kernel, start at once
      int s = 0;
      uint32_t ph = 0;
      for (int kb = kb0; kb < kb1; ++kb) {
        if (!mbar_wait(&emptyW[s], ph ^ 1)) {
          report_error(status, AXB_ERR_WAIT_EMPTY);
          break;
        }
        mbar_expect_tx(&fullW[s], STREAM_W_BYTES);
        tma_load_2d(smem + s * STREAM_W_BYTES, &tmW, &fullW[s], kb * GEMM_BK, m_blk * GEMM_BM);
        if (++s == dw) {
          s = 0;
          ph ^= 1;
        }
      }
    }
  } else if (warp == 6) {
    if (lane == 0) {   // activations: produced by the previous kernel
      grid_dependency_wait();
      int s = 0;
      uint32_t ph = 0;
      for (int kb = kb0; kb < kb1; ++kb) {
        if (!mbar_wait(&emptyX[s], ph ^ 1)) {
          report_error(status, AXB_ERR_WAIT_EMPTY);
          break;
        }
        mbar_expect_tx(&fullX[s], static_cast<uint32_t>(xbytes));
        tma_load_2d(smemX + s * xbytes, &tmX, &fullX[s], kb * GEMM_BK, n_blk * bn);
        if (++s == dx) {
          s = 0;
          ph ^= 1;
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = umma_idesc(GEMM_BM, static_cast<uint32_t>(bn), 0u, 0u);
      int sw = 0, sx = 0;
      uint32_t phw = 0, phx = 0;
      bool issued = kb0 < kb1;
      for (int kb = kb0; kb < kb1; ++kb) {
        if (!mbar_wait(&fullW[sw], phw) || !mbar_wait(&fullX[sx], phx)) {
          report_error(status, AXB_ERR_WAIT_FULL);
          issued = false;
          break;
        }
        tc_fence_after();
        AXB_STL(2, kb == kb0);
        const uint32_t a0 = smem_u32(smem + sw * STREAM_W_BYTES);
        const uint32_t b0 = smem_u32(smemX + sx * xbytes);
#pragma unroll
        for (int j = 0; j < GEMM_BK / 16; ++j)
          umma_f16_ss(tmem_base, umma_smem_desc(a0 + j * 32, 16, 1024), umma_smem_desc(b0 + j * 32, 16, 1024),
                      idesc, (kb != kb0 || j != 0) ? 1u : 0u);
        tc_commit(&emptyW[sw]);
        tc_commit(&emptyX[sx]);
        if (++sw == dw) {
          sw = 0;
          phw ^= 1;
        }
        if (++sx == dx) {
          sx = 0;
          phx ^= 1;
        }
      }
      if (issued) tc_commit(acc_full);
      AXB_STL(3, true);
    }
  } else {
    // ---------------------------------------------------------------- epilogue (warps 2-5, 128 threads)
    grid_dependency_wait();     // before any global write (output, workspace, counters)
    bool ok = kb0 < kb1;
    if (ok && !mbar_wait(acc_full, 0)) {
      report_error(status, AXB_ERR_WAIT_TMEM_FULL);
      ok = false;
    }
    tc_fence_after();
    AXB_STL(4, threadIdx.x == 64);
    const int e = threadIdx.x - 64;
    const int q = warp & 3;
    const int row = q * 32 + lane;                 // feature row inside the tile = TMEM lane
    const int f4 = m_blk * GEMM_BM + (e & 31) * 4;
    const int tok0 = n_blk * bn;
    const int jmax = min(bn, tokens - tok0);       // real tokens of this tile
    const int jpad = (jmax + 15) & ~15;            // accumulator columns read (the padding columns hold zeros)
    const uint32_t t0 = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
    float* stg = reinterpret_cast<float*>(smem);   // the rings are idle once the accumulator is complete
    const int cap_rows = (ring_bytes / (GEMM_BM * 4)) & ~15;   // token rows the staging area holds (multiple of 16)

    if (S == 1) {
      // no split: TMEM -> staging area -> coalesced rows of the output
      for (int r0 = 0; r0 < jpad; r0 += cap_rows) {
        const int rows = min(cap_rows, jpad - r0);
        if (ok) tmem_to_stage<false>(t0, stg, r0, rows, row);
        epi_bar_sync();
        if (ok) stage_to_out(stg, rows, jmax - r0, e, out, ldc, out_fp32, tok0 + r0, f4, feats, false);
        epi_bar_sync();
      }
    } else if (accumulate_mode) {
      float* acc_tile = ws + static_cast<long long>(tile_id) * bn * GEMM_BM;
      unsigned int* tickets = counters + 2 * tile_id;
      unsigned int* done = tickets + 1;
      if (e == 0) *ticket_slot = atomicAdd(tickets, 1u);
      epi_bar_sync();
      const bool last = *ticket_slot == static_cast<uint32_t>(S - 1);
      if (!last) {
        for (int r0 = 0; r0 < jpad; r0 += cap_rows) {
          const int rows = min(cap_rows, jpad - r0);
          if (ok) tmem_to_stage<false>(t0, stg, r0, rows, row);
          fence_async_shared();
          epi_bar_sync();
          if (e == 0) {
            if (ok) bulk_reduce_add_f32(acc_tile + r0 * GEMM_BM, stg, static_cast<uint32_t>(rows * GEMM_BM * 4));
            tma_store_commit();
            tma_store_wait<0>();
          }
          epi_bar_sync();     // staging area reusable, reductions of this chunk complete
        }
        if (e == 0) {
          fence_proxy_async_all();
          __threadfence();
          atomicAdd(done, 1u);
        }
        AXB_STL(5, threadIdx.x == 64);
      } else {
        // last ticket: the other S-1 splits are in their epilogues; wait (bounded) until they are done
        if (e == 0) {
          const long long t_begin = clock64();
          while (ld_acquire_u32(done) < static_cast<unsigned int>(S - 1)) {
            if (clock64() - t_begin > AXB_WAIT_CYCLES) {
              report_error(status, AXB_ERR_WAIT_PEER);
              break;
            }
            __nanosleep(64);
          }
          __threadfence();
          fence_proxy_async_all();
        }
        epi_bar_sync();
        AXB_STL(5, threadIdx.x == 64);
        uint32_t red_phase = 0;
        for (int r0 = 0; r0 < jpad; r0 += cap_rows) {
          const int rows = min(cap_rows, jpad - r0);
          const uint32_t bytes = static_cast<uint32_t>(rows * GEMM_BM * 4);
          if (e == 0) {
            mbar_expect_tx(red_full, bytes);
            bulk_load(stg, acc_tile + r0 * GEMM_BM, bytes, red_full);
          }
          if (!mbar_wait(red_full, red_phase)) report_error(status, AXB_ERR_WAIT_FULL);   // keep going: the barriers below stay matched
          red_phase ^= 1;
          if (ok) tmem_to_stage<true>(t0, stg, r0, rows, row);
          epi_bar_sync();
          stage_to_out(stg, rows, jmax - r0, e, out, ldc, out_fp32, tok0 + r0, f4, feats, true);
          fence_async_shared();
          epi_bar_sync();
          if (e == 0) {
            bulk_store(acc_tile + r0 * GEMM_BM, stg, bytes);      // zeros: the next launch's empty tile
            tma_store_commit();
            tma_store_wait_read<0>();     // the staging area may be reused; the store itself completes by grid end
          }
          epi_bar_sync();
        }
        if (e == 0) {
          *tickets = 0u;
          *done = 0u;
        }
        AXB_STL(6, threadIdx.x == 64);
      }
    } else {
      // bit-reproducible variant: partial tile -> workspace [tile][split][token j][128 feature rows]
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
      if (e == 0) *ticket_slot = atomicAdd(&counters[2 * tile_id], 1u);
      epi_bar_sync();
      AXB_STL(5, threadIdx.x == 64);
      if (*ticket_slot == static_cast<uint32_t>(S - 1)) {
        // last CTA of this tile: sum the S partials in split order, 4 features x 1 token per thread and step
        __threadfence();
        const int l4 = (e & 31) * 4;
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
            if (j < jmax && f4 < feats) {
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
        if (e == 0) counters[2 * tile_id] = 0u;        // ready for the next launch (graph replay)
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
  int bn, tok_tiles, feat_tiles, splits, dw, dx, tmem_cols;
  long long ws_floats;
  int smem_bytes;
};

// planning knobs (changed only by the tuning hook)
static int g_force_splits = 0;        // 0 = heuristic
static int g_max_bn = 128;            // widest token tile
static int g_budget_one = 208 * 1024; // ring bytes when one CTA runs per SM (few tiles)
static int g_budget_two = 104 * 1024; // ring bytes per CTA when two share an SM (many tiles)
static int g_two_tiles = 1;           // from this many output tiles on, two CTAs share an SM (measured: two CTAs with
                                      // twice the splits beat one CTA with a twice as deep ring on every decode shape)
static int g_dx = 0;                  // X ring depth (0: 4 up to 64 tokens, else 3)
static int g_min_kblocks = 8;         // K blocks per split at least
static int g_pdl = 1;                 // launch with programmatic stream serialization
static int g_accumulate = 1;          // split-K partials: 1 = fp32 reductions into one tile, 0 = ordered sum of S tiles

static StreamPlan make_plan(int tokens, int feats, int K) {
  StreamPlan p;
  const int max_bn = g_max_bn < 16 ? 16 : (g_max_bn > 256 ? 256 : g_max_bn / 16 * 16);
  p.tok_tiles = (tokens + max_bn - 1) / max_bn;
  const int per = (tokens + p.tok_tiles - 1) / p.tok_tiles;
  p.bn = (per + 15) / 16 * 16;
  p.feat_tiles = (feats + GEMM_BM - 1) / GEMM_BM;
  const int tiles = p.tok_tiles * p.feat_tiles;
  const int num_k = (K + GEMM_BK - 1) / GEMM_BK;
  const bool two = tiles >= g_two_tiles;
  const int budget = two ? g_budget_two : g_budget_one;
  const int xbytes = p.bn * GEMM_BK * 2;
  p.dx = g_dx > 0 ? g_dx : (p.bn <= 64 ? 4 : 3);
  if (p.dx > STREAM_MAX_X) p.dx = STREAM_MAX_X;
  if (p.dx > num_k) p.dx = num_k;
  if (p.dx < 1) p.dx = 1;
  int dw = (budget - p.dx * xbytes) / STREAM_W_BYTES;
  p.dw = dw < 2 ? 2 : (dw > STREAM_MAX_W ? STREAM_MAX_W : dw);
  p.smem_bytes = p.dw * STREAM_W_BYTES + p.dx * xbytes + STREAM_BAR_BYTES + 1024;
  const int target = two ? 2 * sm_count() : sm_count();
  int s = target / tiles;
  if (s < 1) s = 1;
  const int by_k = num_k / g_min_kblocks;                    // at least this many K blocks per CTA
  if (s > by_k) s = by_k;
  if (s > 16) s = 16;
  if (g_force_splits > 0) s = g_force_splits;
  if (s < 1) s = 1;
  while (s > 1 && (s - 1) * ((num_k + s - 1) / s) >= num_k) --s;   // every split owns at least one K block
  p.splits = s;
  int c = 32;
  while (c < p.bn) c *= 2;
  p.tmem_cols = c;
  p.ws_floats = s > 1 ? static_cast<long long>(tiles) * (g_accumulate ? 1 : s) * p.bn * GEMM_BM : 0;
  return p;
}

}  // namespace axb

#ifdef AXB_TIMELINE
extern "C" int axb_gemm_stream_set_timeline(unsigned long long* buf) {
  return cudaMemcpyToSymbol(axb::g_stream_timeline, &buf, sizeof(buf)) == cudaSuccess ? 0 : -4;
}
#endif

// Tuning hook for experiments. knob: 0 force_splits, 1 max_bn, 2 ring KB (one CTA per SM), 3 ring KB (two per SM),
// 4 tile count from which two CTAs share an SM, 5 X ring depth, 6 min K blocks per split, 7 dependent launch,
// 8 accumulate (1) / ordered (0) split-K. Returns the previous value.
extern "C" int axb_gemm_stream_knob(int knob, int value) {
  using namespace axb;
  int* slot[] = {&g_force_splits, &g_max_bn, &g_budget_one, &g_budget_two, &g_two_tiles, &g_dx, &g_min_kblocks, &g_pdl, &g_accumulate};
  if (knob < 0 || knob > 8) return -1;
  const int scale = (knob == 2 || knob == 3) ? 1024 : 1;
  const int old = *slot[knob] / scale;
  *slot[knob] = value * scale;
  return old;
}

// Workspace the launch of this shape needs: fp32 elements of partial tiles (0 without a K split) and the
// number of 32-bit counters (zero-initialised once by the caller, self-resetting afterwards).
// `zeroed` = 1: the fp32 workspace must be all zero before the first launch (every launch leaves it zero again).
extern "C" int axb_gemm_stream_workspace(int tokens, int feats, int K, long long* ws_floats, int* n_counters,
                                         int* splits, int* bn, int* zeroed) {
  using namespace axb;
  if (tokens <= 0 || feats <= 0 || K <= 0) return AXB_LAUNCH_BAD_ARG;
  const StreamPlan p = make_plan(tokens, feats, K);
  if (ws_floats) *ws_floats = p.ws_floats;
  if (n_counters) *n_counters = 2 * p.tok_tiles * p.feat_tiles;
  if (splits) *splits = p.splits;
  if (bn) *bn = p.bn;
  if (zeroed) *zeroed = g_accumulate;
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
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(p.splits, p.feat_tiles, p.tok_tiles);
  cfg.blockDim = dim3(STREAM_THREADS, 1, 1);
  cfg.dynamicSmemBytes = p.smem_bytes;
  cfg.stream = static_cast<cudaStream_t>(stream);
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = g_pdl ? 1 : 0;
  if (cudaLaunchKernelEx(&cfg, gemm_stream_kernel, tmW, tmX, feats, tokens, K, p.bn, p.dw, p.dx, p.tmem_cols, ws,
                         counters, out, ldc, out_fp32, g_accumulate, status) != cudaSuccess) {
    cudaGetLastError();
    return AXB_LAUNCH_CUDA_ERROR;
  }
  return check_launch();
}
