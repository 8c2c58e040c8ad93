// Persistent warp-specialised tcgen05 GEMM core for sm_100a.
//
//   D[M,N] = A[M,K] * B[N,K]^T     (fp32 accumulation in TMEM)
//
// One CTA per SM, 192 threads:
//   warp 0     TMA producer   (cp.async.bulk.tensor 2-D, 128-byte swizzle, no multicast)
//   warp 1     MMA issuer     (one lane issues tcgen05.mma; owns TMEM alloc/dealloc)
//   warps 2-5  epilogue       (tcgen05.ld 32x32b: thread t of a warp owns one output row)
// The accumulator is double-buffered in TMEM (2 x BN columns) so the epilogue of tile i
// overlaps the main loop of tile i+1. Tiles are 128 x BN with BK = 64 (one 128-byte swizzle
// atom of bf16 along the contiguous dimension).
//
// Each operand may be K-major (rows are M/N, K contiguous) or MN-major (rows are K, M/N
// contiguous), which gives NN/NT/TN/TT products without a transpose pass:
//   forward   Y = X W^T      : A = X  (K-major),  B = W  (K-major)
//   dgrad     dX = dY W      : A = dY (K-major),  B = W  (MN-major)
//   wgrad     dW = dY^T X    : A = dY (MN-major), B = X  (MN-major)
//
// The epilogue is a functor so fused consumers (bf16/fp32 store, accumulate, SwiGLU,
// soft-max statistics for the vocabulary head, ...) share the main loop.
#pragma once
#include "ptx.cuh"
#include <cuda.h>

namespace axb {

constexpr int GEMM_BM = 128;
constexpr int GEMM_BK = 64;
constexpr int GEMM_THREADS = 192;
constexpr int GEMM_GROUP_M = 8;

template <int BN>
struct GemmSmem {
  static constexpr int A_BYTES = GEMM_BM * GEMM_BK * 2;
  static constexpr int B_BYTES = BN * GEMM_BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  // Leave room for barriers and the 1024-byte alignment slack inside 227 KB.
  static constexpr int STAGES = (BN == 256) ? 4 : (BN == 128 ? 6 : 8);
  static constexpr int BAR_BYTES = 256;
  static constexpr int TOTAL = STAGES * STAGE_BYTES + BAR_BYTES + 1024;
};

struct GemmShape {
  int M, N, K;
  int k_splits;  // >= 1; split s handles K blocks [s*kper, (s+1)*kper) and the epilogue receives s
};

__device__ __forceinline__ void tile_coords(int t, int num_m, int num_n, int k_splits, int& m_blk,
                                            int& n_blk, int& split) {
  split = t % k_splits;  // splits of one output tile run side by side
  t /= k_splits;
  const int group = GEMM_GROUP_M * num_n;
  const int gid = t / group;
  const int first_m = gid * GEMM_GROUP_M;
  const int gm = min(num_m - first_m, GEMM_GROUP_M);
  const int r = t - gid * group;
  m_blk = first_m + (r % gm);
  n_blk = r / gm;
}

// Tile maps: which (m, n, split) tile a linear tile index denotes, which K blocks it covers and
// where its B rows and output rows start. The dense map is the plain rasterisation above; the two
// grouped maps serve mixture-of-experts layers whose rows are sorted by expert and padded to 128.
struct TileInfo {
  int m_blk, n_blk, split;
  int kb0, kb1;     // K blocks [kb0, kb1)
  int b_off;        // added to B's outer (row) coordinate: expert * rows-per-expert
  int epi_m_blk;    // row block the epilogue writes
  bool valid;
};

struct DenseTiles {
  static constexpr bool PEER_A = false;
  struct Params {};
  __device__ static int rows(const Params&, const GemmShape& sh) { return sh.M; }
  __device__ static int epi_rows(const Params&, const GemmShape& sh) { return sh.M; }
  __device__ static int num_tiles(const Params&, const GemmShape& sh, int num_m, int num_n) {
    return num_m * num_n * (sh.k_splits < 1 ? 1 : sh.k_splits);
  }
  __device__ static TileInfo decode(const Params&, const GemmShape& sh, int t, int num_m, int num_n, int num_k) {
    TileInfo ti;
    const int ks = sh.k_splits < 1 ? 1 : sh.k_splits;
    tile_coords(t, num_m, num_n, ks, ti.m_blk, ti.n_blk, ti.split);
    const int k_per = (num_k + ks - 1) / ks;
    ti.kb0 = ti.split * k_per;
    ti.kb1 = min(num_k, ti.kb0 + k_per);
    ti.b_off = 0;
    ti.epi_m_blk = ti.m_blk;
    ti.valid = true;
    return ti;
  }
};

// Rows of A / C are sorted by expert (128-row aligned); B holds E stacked weight matrices. Every
// 128-row block belongs to one expert (tile_expert[m]); the number of live rows is read on the device.
struct RowGroupedTiles {
  static constexpr bool PEER_A = false;
  struct Params {
    const int* tile_expert;
    const int* total_rows;     // offsets[E]: padded row count actually in use
    int b_rows_per_expert;
  };
  __device__ static int rows(const Params& p, const GemmShape& sh) { return min(sh.M, *p.total_rows); }
  __device__ static int epi_rows(const Params& p, const GemmShape& sh) { return min(sh.M, *p.total_rows); }
  __device__ static int num_tiles(const Params&, const GemmShape&, int num_m, int num_n) { return num_m * num_n; }
  __device__ static TileInfo decode(const Params& p, const GemmShape&, int t, int num_m, int num_n, int num_k) {
    TileInfo ti;
    tile_coords(t, num_m, num_n, 1, ti.m_blk, ti.n_blk, ti.split);
    const int e = p.tile_expert[ti.m_blk];
    ti.kb0 = 0;
    ti.kb1 = num_k;
    ti.b_off = (e < 0 ? 0 : e) * p.b_rows_per_expert;
    ti.epi_m_blk = ti.m_blk;
    ti.valid = e >= 0;
    return ti;
  }
};

// Per-expert weight gradients: the contraction runs over the rows of one expert (a K range), the
// output is that expert's [M, N] slice of a stacked [E*M, N] tensor.
struct KGroupedTiles {
  static constexpr bool PEER_A = false;
  struct Params {
    const int* offsets;        // [E + 1] row offsets (multiples of 128)
    int num_experts;
  };
  __device__ static int rows(const Params&, const GemmShape& sh) { return sh.M; }
  __device__ static int epi_rows(const Params& p, const GemmShape& sh) { return sh.M * p.num_experts; }
  __device__ static int num_tiles(const Params& p, const GemmShape&, int num_m, int num_n) {
    return p.num_experts * num_m * num_n;
  }
  __device__ static TileInfo decode(const Params& p, const GemmShape&, int t, int num_m, int num_n, int) {
    TileInfo ti;
    const int per = num_m * num_n;
    const int e = t / per;
    tile_coords(t - e * per, num_m, num_n, 1, ti.m_blk, ti.n_blk, ti.split);
    ti.kb0 = p.offsets[e] / GEMM_BK;
    ti.kb1 = p.offsets[e + 1] / GEMM_BK;
    ti.b_off = 0;
    ti.epi_m_blk = e * num_m + ti.m_blk;
    ti.valid = ti.kb1 > ti.kb0;
    return ti;
  }
};

// All-gather fused into the GEMM: A is row-sharded over `world` ranks (sequence-parallel activations in
// symmetric memory); row block m lives on rank m / blocks_per_rank. Each A tile is fetched by TMA
// straight from its owner's buffer (plain, non-multicast loads over NVLink) — no gathered copy exists.
// Blocks are visited starting with this rank's own rows, then the next rank's, so the ranks do not all
// pull from the same peer at the same time.
struct PeerGatherTiles {
  static constexpr bool PEER_A = true;
  static constexpr int MAX_RANKS = 8;
  struct Params {
    CUtensorMap maps[MAX_RANKS];   // map r describes rank r's shard [rows_per_rank][K]
    int world, rank, blocks_per_rank;
  };
  __device__ static int rows(const Params&, const GemmShape& sh) { return sh.M; }
  __device__ static int epi_rows(const Params&, const GemmShape& sh) { return sh.M; }
  __device__ static int num_tiles(const Params&, const GemmShape&, int num_m, int num_n) { return num_m * num_n; }
  __device__ static TileInfo decode(const Params& p, const GemmShape&, int t, int num_m, int num_n, int num_k) {
    TileInfo ti;
    tile_coords(t, num_m, num_n, 1, ti.m_blk, ti.n_blk, ti.split);
    ti.m_blk = (ti.m_blk + p.rank * p.blocks_per_rank) % num_m;      // own rows first
    ti.kb0 = 0;
    ti.kb1 = num_k;
    ti.b_off = 0;
    ti.epi_m_blk = ti.m_blk;
    ti.valid = true;
    return ti;
  }
  __device__ static const CUtensorMap* a_map(const Params& p, int m_blk) { return &p.maps[m_blk / p.blocks_per_rank]; }
  __device__ static int a_row(const Params& p, int m_blk) { return (m_blk % p.blocks_per_rank) * GEMM_BM; }
};

// Epi contract:
//   struct Params;                                   // POD passed by value
//   __device__ Epi(const Params&, int m_blk, int n_blk, int row, const GemmShape&, int split);
//   __device__ void chunk(int col0, const uint32_t (&acc)[32]);   // 32 fp32 columns of `row`
//   __device__ void finish();
template <int BN, bool A_MN, bool B_MN, class Epi, class TM = DenseTiles>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
               const GemmShape shape, const typename Epi::Params ep, int* status,
               const __grid_constant__ typename TM::Params tp) {
  using S = GemmSmem<BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + S::STAGES * S::STAGE_BYTES);
  uint64_t* full = bars;                      // [STAGES]
  uint64_t* empty = bars + S::STAGES;         // [STAGES]
  uint64_t* acc_full = bars + 2 * S::STAGES;  // [2]
  uint64_t* acc_empty = acc_full + 2;         // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_m = (TM::rows(tp, shape) + GEMM_BM - 1) / GEMM_BM;
  const int num_n = (shape.N + BN - 1) / BN;
  const int num_k_total = (shape.K + GEMM_BK - 1) / GEMM_BK;
  const int num_tiles = TM::num_tiles(tp, shape, num_m, num_n);
  GemmShape epi_shape = shape;
  epi_shape.M = TM::epi_rows(tp, shape);
  constexpr uint32_t TMEM_COLS = 2 * BN < 32 ? 32 : 2 * BN;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S::STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 128);
    }
    mbar_fence_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        const TileInfo ti = TM::decode(tp, shape, t, num_m, num_n, num_k_total);
        if (!ti.valid) continue;
        const int m_blk = ti.m_blk, n_blk = ti.n_blk;
        const int kb0 = ti.kb0, kb1 = ti.kb1;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&empty[s], ph ^ 1)) {
            report_error(status, AXB_ERR_WAIT_EMPTY);
            ok = false;
            break;
          }
          uint8_t* sA = smem + s * S::STAGE_BYTES;
          uint8_t* sB = sA + S::A_BYTES;
          mbar_expect_tx(&full[s], S::STAGE_BYTES);
          if constexpr (TM::PEER_A) {
            static_assert(!TM::PEER_A || !A_MN, "peer-gathered A operands are K-major");
            tma_load_2d(sA, TM::a_map(tp, m_blk), &full[s], kb * GEMM_BK, TM::a_row(tp, m_blk));
          } else if (!A_MN) {
            tma_load_2d(sA, &tmA, &full[s], kb * GEMM_BK, m_blk * GEMM_BM);
          } else {
#pragma unroll
            for (int c = 0; c < GEMM_BM / 64; ++c)
              tma_load_2d(sA + c * 8192, &tmA, &full[s], m_blk * GEMM_BM + c * 64, kb * GEMM_BK);
          }
          if (!B_MN) {
            tma_load_2d(sB, &tmB, &full[s], kb * GEMM_BK, n_blk * BN + ti.b_off);
          } else {
#pragma unroll
            for (int c = 0; c < BN / 64; ++c)
              tma_load_2d(sB + c * 8192, &tmB, &full[s], n_blk * BN + c * 64, kb * GEMM_BK + ti.b_off);
          }
          if (++s == S::STAGES) {
            s = 0;
            ph ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc(GEMM_BM, BN, A_MN ? 1u : 0u, B_MN ? 1u : 0u);
      int s = 0;
      uint32_t ph = 0;
      int it = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        const TileInfo ti = TM::decode(tp, shape, t, num_m, num_n, num_k_total);
        if (!ti.valid) continue;
        const int buf = it & 1;
        if (!mbar_wait(&acc_empty[buf], ((it >> 1) & 1) ^ 1)) {
          report_error(status, AXB_ERR_WAIT_TMEM_EMPTY);
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * BN;
        const int kb0 = ti.kb0, kb1 = ti.kb1;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&full[s], ph)) {
            report_error(status, AXB_ERR_WAIT_FULL);
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a0 = smem_u32(smem + s * S::STAGE_BYTES);
          const uint32_t b0 = a0 + S::A_BYTES;
#pragma unroll
          for (int j = 0; j < GEMM_BK / 16; ++j) {
            const uint64_t ad = A_MN ? umma_smem_desc(a0 + j * 2048, 8192, 1024)
                                     : umma_smem_desc(a0 + j * 32, 16, 1024);
            const uint64_t bd = B_MN ? umma_smem_desc(b0 + j * 2048, 8192, 1024)
                                     : umma_smem_desc(b0 + j * 32, 16, 1024);
            umma_f16_ss(d_tmem, ad, bd, idesc, (kb != kb0 || j != 0) ? 1u : 0u);
          }
          tc_commit(&empty[s]);
          if (++s == S::STAGES) {
            s = 0;
            ph ^= 1;
          }
        }
        if (ok) tc_commit(&acc_full[buf]);
        ++it;
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    int it = 0;
    for (int t = blockIdx.x; t < num_tiles; t += gridDim.x) {
      const TileInfo ti = TM::decode(tp, shape, t, num_m, num_n, num_k_total);
      if (!ti.valid) continue;
      const int m_blk = ti.epi_m_blk, n_blk = ti.n_blk, split = ti.split;
      const int buf = it & 1;
      if (!mbar_wait(&acc_full[buf], (it >> 1) & 1)) {
        report_error(status, AXB_ERR_WAIT_TMEM_FULL);
        break;
      }
      tc_fence_after();
      const int row = m_blk * GEMM_BM + q * 32 + lane;
      Epi epi(ep, m_blk, n_blk, row, epi_shape, split);
      const uint32_t t0 = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + buf * BN;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t acc[32];
        tmem_ld_32x32(t0 + c * 32, acc);
        tmem_ld_wait();
        epi.chunk(n_blk * BN + c * 32, acc);
      }
      tc_fence_before();
      mbar_arrive(&acc_empty[buf]);
      epi.finish();
      ++it;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ------------------------------------------------------------------------- store epilogue
// mode 0: bf16 store, 1: fp32 store, 2: fp32 accumulate (C += acc), 3: bf16 accumulate.
// alpha scales the accumulator first.
struct StoreEpi {
  struct Params {
    void* C;
    long long ldc;
    int mode;
    float alpha;
  };
  const Params& p;
  const GemmShape& sh;
  int row;
  __device__ StoreEpi(const Params& p_, int, int, int row_, const GemmShape& sh_, int)
      : p(p_), sh(sh_), row(row_) {}
  __device__ __forceinline__ void chunk(int col0, const uint32_t (&acc)[32]) {
    if (row >= sh.M || col0 >= sh.N) return;
    const bool full = (col0 + 32 <= sh.N) && ((p.ldc & 7) == 0);
    const float a = p.alpha;
    if (p.mode == 0) {
      __nv_bfloat16* c = reinterpret_cast<__nv_bfloat16*>(p.C) + (long long)row * p.ldc + col0;
      if (full) {
#pragma unroll
        for (int v = 0; v < 4; ++v) {
          uint4 o;
          o.x = pack_bf16x2(__uint_as_float(acc[8 * v + 0]) * a, __uint_as_float(acc[8 * v + 1]) * a);
          o.y = pack_bf16x2(__uint_as_float(acc[8 * v + 2]) * a, __uint_as_float(acc[8 * v + 3]) * a);
          o.z = pack_bf16x2(__uint_as_float(acc[8 * v + 4]) * a, __uint_as_float(acc[8 * v + 5]) * a);
          o.w = pack_bf16x2(__uint_as_float(acc[8 * v + 6]) * a, __uint_as_float(acc[8 * v + 7]) * a);
          reinterpret_cast<uint4*>(c)[v] = o;
        }
      } else {
        for (int j = 0; j < 32 && col0 + j < sh.N; ++j)
          c[j] = __float2bfloat16(__uint_as_float(acc[j]) * a);
      }
    } else if (p.mode == 3) {
      __nv_bfloat16* c = reinterpret_cast<__nv_bfloat16*>(p.C) + (long long)row * p.ldc + col0;
      for (int j = 0; j < 32 && col0 + j < sh.N; ++j)
        c[j] = __float2bfloat16(__bfloat162float(c[j]) + __uint_as_float(acc[j]) * a);
    } else {
      float* c = reinterpret_cast<float*>(p.C) + (long long)row * p.ldc + col0;
      const bool accum = p.mode == 2;
      if (full && (p.ldc & 3) == 0) {
#pragma unroll
        for (int v = 0; v < 8; ++v) {
          float4 o = make_float4(__uint_as_float(acc[4 * v + 0]) * a, __uint_as_float(acc[4 * v + 1]) * a,
                                 __uint_as_float(acc[4 * v + 2]) * a, __uint_as_float(acc[4 * v + 3]) * a);
          if (accum) {
            const float4 old = reinterpret_cast<float4*>(c)[v];
            o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
          }
          reinterpret_cast<float4*>(c)[v] = o;
        }
      } else {
        for (int j = 0; j < 32 && col0 + j < sh.N; ++j) {
          const float v = __uint_as_float(acc[j]) * a;
          c[j] = accum ? c[j] + v : v;
        }
      }
    }
  }
  __device__ __forceinline__ void finish() {}
};

// ------------------------------------------------------------------------- peer scatter epilogue
// Reduce-scatter fused into the GEMM: every rank computes a partial [T][N]; the rows are owned by
// rank row / rows_per_rank. The epilogue stores each 128 x 32 piece, as bf16, straight into the owner's
// staging area slot [source rank][local row][N] with plain peer stores, so the NVLink transfer runs tile
// by tile underneath the remaining MMAs. A barrier and a fixed-order sum over the slots finish it.
struct PeerScatterEpi {
  static constexpr int MAX_RANKS = 8;
  struct Params {
    void* staging[MAX_RANKS];   // rank r's staging buffer: [world][rows_per_rank][ld] bf16
    long long ld;
    int rows_per_rank, rank;
  };
  const Params& p;
  const GemmShape& sh;
  int row;
  __device__ PeerScatterEpi(const Params& p_, int, int, int row_, const GemmShape& sh_, int)
      : p(p_), sh(sh_), row(row_) {}
  __device__ __forceinline__ void chunk(int col0, const uint32_t (&acc)[32]) {
    if (row >= sh.M || col0 >= sh.N) return;
    const int owner = row / p.rows_per_rank;
    const int local = row - owner * p.rows_per_rank;
    __nv_bfloat16* c = reinterpret_cast<__nv_bfloat16*>(p.staging[owner]) +
                       (static_cast<long long>(p.rank) * p.rows_per_rank + local) * p.ld + col0;
    if (col0 + 32 <= sh.N && (p.ld & 7) == 0) {
#pragma unroll
      for (int v = 0; v < 4; ++v) {
        uint4 o;
        o.x = pack_bf16x2(__uint_as_float(acc[8 * v + 0]), __uint_as_float(acc[8 * v + 1]));
        o.y = pack_bf16x2(__uint_as_float(acc[8 * v + 2]), __uint_as_float(acc[8 * v + 3]));
        o.z = pack_bf16x2(__uint_as_float(acc[8 * v + 4]), __uint_as_float(acc[8 * v + 5]));
        o.w = pack_bf16x2(__uint_as_float(acc[8 * v + 6]), __uint_as_float(acc[8 * v + 7]));
        reinterpret_cast<uint4*>(c)[v] = o;
      }
    } else {
      for (int j = 0; j < 32 && col0 + j < sh.N; ++j) c[j] = __float2bfloat16(__uint_as_float(acc[j]));
    }
  }
  __device__ __forceinline__ void finish() {}
};

// ------------------------------------------------------------------------- transposed epilogue
// For "swap-AB" products (weights as the 128-row operand, a small token batch as the N operand):
// the accumulator row is an output FEATURE and the column a TOKEN, so element (row, col) goes to
// C[col][row]. Lanes of a warp hold consecutive rows, hence each store instruction writes 32
// consecutive elements of one token row. With k_splits > 1 fp32 partials go to
// ws[split][token][feature] and a reduce kernel finishes; with one split the final dtype is written.
struct TransposedEpi {
  struct Params {
    void* C;          // [tokens][ldc] bf16 (mode 0) or fp32 (mode 1)
    long long ldc;
    int mode;
    float* ws;        // [k_splits][tokens][features] fp32, used when k_splits > 1
  };
  const Params& p;
  const GemmShape& sh;
  int row, split;
  __device__ TransposedEpi(const Params& p_, int, int, int row_, const GemmShape& sh_, int split_)
      : p(p_), sh(sh_), row(row_), split(split_) {}
  __device__ __forceinline__ void chunk(int col0, const uint32_t (&acc)[32]) {
    if (row >= sh.M || col0 >= sh.N) return;
    if (sh.k_splits > 1) {
      float* w = p.ws + ((long long)split * sh.N + col0) * sh.M + row;
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (col0 + j < sh.N) w[(long long)j * sh.M] = __uint_as_float(acc[j]);
    } else if (p.mode == 0) {
      __nv_bfloat16* c = reinterpret_cast<__nv_bfloat16*>(p.C) + (long long)col0 * p.ldc + row;
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (col0 + j < sh.N) c[(long long)j * p.ldc] = __float2bfloat16(__uint_as_float(acc[j]));
    } else {
      float* c = reinterpret_cast<float*>(p.C) + (long long)col0 * p.ldc + row;
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (col0 + j < sh.N) c[(long long)j * p.ldc] = __uint_as_float(acc[j]);
    }
  }
  __device__ __forceinline__ void finish() {}
};

}  // namespace axb
