// extern "C" launchers for the plain bf16 GEMM built on gemm_core.cuh.
#include "gemm_core.cuh"
#include "host_utils.h"

namespace axb {

// b_rows / a_rows: outer extents of the tensor maps (rows of the operand matrices as stored); they
// differ from N / M for stacked expert weights and expert-sorted activations.
template <int BN, bool A_MN, bool B_MN, class Epi, class TM = DenseTiles>
static int launch_gemm_inst(const void* A, const void* B, int M, int N, int K, long long lda,
                            long long ldb, const typename Epi::Params& ep, int* status,
                            cudaStream_t stream, int max_ctas, int k_splits = 1,
                            const typename TM::Params& tp = typename TM::Params{}, long long a_rows = -1,
                            long long b_rows = -1, int tiles_hint = -1) {
  CUtensorMap tmA, tmB;
  int rc;
  // K-major operand: tensor [rows][K]; MN-major operand: tensor [K rows][M or N]
  const long long a_outer = a_rows >= 0 ? a_rows : (A_MN ? K : M);
  const long long b_outer = b_rows >= 0 ? b_rows : (B_MN ? K : N);
  if (!A_MN)
    rc = make_tmap_2d(&tmA, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, a_outer, lda * 2, GEMM_BK, GEMM_BM, true);
  else
    rc = make_tmap_2d(&tmA, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, M, a_outer, lda * 2, 64, GEMM_BK, true);
  if (rc != AXB_LAUNCH_OK) return rc;
  if (!B_MN)
    rc = make_tmap_2d(&tmB, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, b_outer, ldb * 2, GEMM_BK, BN, true);
  else
    rc = make_tmap_2d(&tmB, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, N, b_outer, ldb * 2, 64, GEMM_BK, true);
  if (rc != AXB_LAUNCH_OK) return rc;

  auto kern = gemm_tc_kernel<BN, A_MN, B_MN, Epi, TM>;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             GemmSmem<BN>::TOTAL) != cudaSuccess)
      return AXB_LAUNCH_CUDA_ERROR;
    attr_set = true;
  }
  const int num_tiles = ((M + GEMM_BM - 1) / GEMM_BM) * ((N + BN - 1) / BN);
  const int num_tiles_k = tiles_hint > 0 ? tiles_hint : num_tiles * (k_splits < 1 ? 1 : k_splits);
  int grid = sm_count();
  if (max_ctas > 0 && max_ctas < grid) grid = max_ctas;
  if (num_tiles_k < grid) grid = num_tiles_k;
  GemmShape sh{M, N, K, k_splits < 1 ? 1 : k_splits};
  kern<<<grid, GEMM_THREADS, GemmSmem<BN>::TOTAL, stream>>>(tmA, tmB, sh, ep, status, tp);
  return check_launch();
}

template <class Epi>
static int launch_gemm(const void* A, const void* B, int M, int N, int K, long long lda,
                       long long ldb, int a_mn, int b_mn, const typename Epi::Params& ep,
                       int* status, cudaStream_t stream, int bn_hint, int max_ctas) {
  if (M <= 0 || N <= 0 || K <= 0) return AXB_LAUNCH_BAD_ARG;
  // Tile width: the widest tile that still gives every SM work.
  int bn = bn_hint;
  if (bn != 64 && bn != 128 && bn != 256) {
    const int sms = sm_count();
    const long long mt = (M + GEMM_BM - 1) / GEMM_BM;
    if (mt * ((N + 255) / 256) >= sms) bn = 256;
    else if (mt * ((N + 127) / 128) >= sms) bn = 128;
    else bn = 64;
    if (N <= 64) bn = 64;
  }
#define AXB_DISPATCH(BN_)                                                                      \
  do {                                                                                         \
    if (!a_mn && !b_mn)                                                                        \
      return launch_gemm_inst<BN_, false, false, Epi>(A, B, M, N, K, lda, ldb, ep, status, stream, max_ctas); \
    if (!a_mn && b_mn)                                                                         \
      return launch_gemm_inst<BN_, false, true, Epi>(A, B, M, N, K, lda, ldb, ep, status, stream, max_ctas);  \
    if (a_mn && !b_mn)                                                                         \
      return launch_gemm_inst<BN_, true, false, Epi>(A, B, M, N, K, lda, ldb, ep, status, stream, max_ctas);  \
    return launch_gemm_inst<BN_, true, true, Epi>(A, B, M, N, K, lda, ldb, ep, status, stream, max_ctas);     \
  } while (0)
  if (bn == 256) AXB_DISPATCH(256);
  if (bn == 128) AXB_DISPATCH(128);
  AXB_DISPATCH(64);
#undef AXB_DISPATCH
}

// out[t][f] = sum_s ws[s][t][f]  (fp32 partials of a split-K product), bf16 or fp32 result
__global__ void splitk_reduce_kernel(const float* __restrict__ ws, void* __restrict__ out, long long ldc,
                                     int tokens, int feats, int splits, int out_fp32) {
  const long long n = (long long)tokens * feats;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    float acc = 0.f;
    for (int s = 0; s < splits; ++s) acc += ws[(long long)s * n + i];
    const long long t = i / feats, f = i - t * feats;
    if (out_fp32) reinterpret_cast<float*>(out)[t * ldc + f] = acc;
    else reinterpret_cast<__nv_bfloat16*>(out)[t * ldc + f] = __float2bfloat16(acc);
  }
}

}  // namespace axb

// C[M,N] (=|+=) alpha * op(A) op(B)^T.
//   a_mn = 0: A is [M][lda] (K contiguous);  a_mn = 1: A is [K][lda] (M contiguous)
//   b_mn = 0: B is [N][ldb] (K contiguous);  b_mn = 1: B is [K][ldb] (N contiguous)
//   out_mode 0 bf16 store, 1 fp32 store, 2 fp32 accumulate, 3 bf16 accumulate.
// Leading dimensions are in elements and must be multiples of 8; base pointers 16-byte aligned.
extern "C" int axb_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K,
                             long long lda, long long ldb, long long ldc, int a_mn, int b_mn,
                             int out_mode, float alpha, int bn_hint, int max_ctas, int* status,
                             void* stream) {
  using namespace axb;
  if ((lda & 7) || (ldb & 7) || out_mode < 0 || out_mode > 3) return AXB_LAUNCH_BAD_ARG;
  if ((reinterpret_cast<uintptr_t>(C) & 15) != 0) return AXB_LAUNCH_BAD_ARG;
  StoreEpi::Params ep{C, ldc, out_mode, alpha};
  return launch_gemm<StoreEpi>(A, B, M, N, K, lda, ldb, a_mn, b_mn, ep, status,
                               static_cast<cudaStream_t>(stream), bn_hint, max_ctas);
}

// Number of K splits the small-batch product will use (the caller sizes the workspace with it).
extern "C" int axb_gemm_smallm_splits(int tokens, int feats, int K) {
  using namespace axb;
  const int bn = tokens <= 64 ? 64 : (tokens <= 128 ? 128 : 256);
  const int tiles = ((feats + GEMM_BM - 1) / GEMM_BM) * ((tokens + bn - 1) / bn);
  const int num_k = (K + GEMM_BK - 1) / GEMM_BK;
  const int sms = sm_count();
  if (tiles >= sms) return 1;
  int splits = (sms + tiles - 1) / tiles;
  const int max_splits = num_k / 8 > 0 ? num_k / 8 : 1;  // keep at least 8 K blocks per split
  if (splits > max_splits) splits = max_splits;
  if (splits > 16) splits = 16;
  return splits < 1 ? 1 : splits;
}

// Small token batch ("swap-AB"): out[tokens][feats] = X[tokens][K] * W[feats][K]^T with the weight
// rows on the 128-wide MMA M side, so the weights stream once at full tile efficiency, plus split-K
// to occupy every SM. ws: fp32 [splits][tokens][feats] (splits from axb_gemm_smallm_splits), may be
// null when that returns 1. out_fp32 selects fp32 (logits) or bf16 output.
extern "C" int axb_gemm_bf16_smallm(const void* X, const void* W, void* out, int tokens, int feats, int K,
                                    long long ldx, long long ldw, long long ldc, int out_fp32, float* ws,
                                    int* status, void* stream) {
  using namespace axb;
  if (tokens <= 0 || feats <= 0 || K <= 0 || (ldx & 7) || (ldw & 7)) return AXB_LAUNCH_BAD_ARG;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int splits = axb_gemm_smallm_splits(tokens, feats, K);
  if (splits > 1 && ws == nullptr) return AXB_LAUNCH_BAD_ARG;
  TransposedEpi::Params ep{out, ldc, out_fp32 ? 1 : 0, ws};
  int rc;
  if (tokens <= 64)
    rc = launch_gemm_inst<64, false, false, TransposedEpi>(W, X, feats, tokens, K, ldw, ldx, ep, status, s, 0, splits);
  else if (tokens <= 128)
    rc = launch_gemm_inst<128, false, false, TransposedEpi>(W, X, feats, tokens, K, ldw, ldx, ep, status, s, 0, splits);
  else
    rc = launch_gemm_inst<256, false, false, TransposedEpi>(W, X, feats, tokens, K, ldw, ldx, ep, status, s, 0, splits);
  if (rc || splits == 1) return rc;
  const long long n = (long long)tokens * feats;
  long long blocks = (n + 255) / 256;
  const long long cap = (long long)sm_count() * 8;
  if (blocks > cap) blocks = cap;
  splitk_reduce_kernel<<<(int)blocks, 256, 0, s>>>(ws, out, ldc, tokens, feats, splits, out_fp32);
  return check_launch();
}


// ------------------------------------------------------------------ grouped (mixture-of-experts)
// Rows of X / Y are sorted by expert and padded to 128 per expert (see moe.cu):
//   tile_expert[m]  expert of 128-row block m (-1 past the end);  total_rows = padded rows in use.
// forward   Y[P][N]  = X[P][K]  * W_e[N][K]^T          (W stacked [E*N][K])
// dgrad     dX[P][K] = dY[P][N] * W_e[N][K]            (same W, read MN-major)
// wgrad     dW_e[N][K] += dY_e^T X_e  in fp32          (contraction over the expert's rows)
// P = max_rows (capacity of the sorted buffers). N and K of the weights must be multiples of 128.
extern "C" int axb_gemm_grouped_fwd(const void* X, const void* W, void* Y, int max_rows, int N, int K, int E,
                                    long long ldx, long long ldw, long long ldy, const int* tile_expert,
                                    const int* total_rows, int* status, void* stream) {
  using namespace axb;
  if (max_rows <= 0 || N % 128 != 0 || K % 64 != 0 || E <= 0 || (ldx & 7) || (ldw & 7)) return AXB_LAUNCH_BAD_ARG;
  StoreEpi::Params ep{Y, ldy, 0, 1.0f};
  RowGroupedTiles::Params tp{tile_expert, total_rows, N};
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (N % 256 == 0)
    return launch_gemm_inst<256, false, false, StoreEpi, RowGroupedTiles>(X, W, max_rows, N, K, ldx, ldw, ep, status, s,
                                                                           0, 1, tp, max_rows, (long long)E * N);
  return launch_gemm_inst<128, false, false, StoreEpi, RowGroupedTiles>(X, W, max_rows, N, K, ldx, ldw, ep, status, s, 0,
                                                                         1, tp, max_rows, (long long)E * N);
}

// dX[P][Kw] = dY[P][Nw] * W_e[Nw][Kw]: GEMM with N_gemm = Kw, K_gemm = Nw, B MN-major, rows of B offset by e*Nw.
extern "C" int axb_gemm_grouped_dgrad(const void* dY, const void* W, void* dX, int max_rows, int Nw, int Kw, int E,
                                      long long lddy, long long ldw, long long lddx, const int* tile_expert,
                                      const int* total_rows, int* status, void* stream) {
  using namespace axb;
  if (max_rows <= 0 || Nw % 64 != 0 || Kw % 128 != 0 || E <= 0 || (lddy & 7) || (ldw & 7)) return AXB_LAUNCH_BAD_ARG;
  StoreEpi::Params ep{dX, lddx, 0, 1.0f};
  RowGroupedTiles::Params tp{tile_expert, total_rows, Nw};
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (Kw % 256 == 0)
    return launch_gemm_inst<256, false, true, StoreEpi, RowGroupedTiles>(dY, W, max_rows, Kw, Nw, lddy, ldw, ep, status, s,
                                                                          0, 1, tp, max_rows, (long long)E * Nw);
  return launch_gemm_inst<128, false, true, StoreEpi, RowGroupedTiles>(dY, W, max_rows, Kw, Nw, lddy, ldw, ep, status, s, 0,
                                                                        1, tp, max_rows, (long long)E * Nw);
}

// dW[E][Nw][Kw] (fp32) += dY_e^T X_e. offsets: [E+1] row offsets of the experts (device).
extern "C" int axb_gemm_grouped_wgrad(const void* dY, const void* X, float* dW, int max_rows, int Nw, int Kw, int E,
                                      long long lddy, long long ldx, const int* offsets, int accumulate, int* status,
                                      void* stream) {
  using namespace axb;
  if (max_rows <= 0 || Nw % 128 != 0 || Kw % 128 != 0 || E <= 0 || (lddy & 7) || (ldx & 7)) return AXB_LAUNCH_BAD_ARG;
  StoreEpi::Params ep{dW, Kw, accumulate ? 2 : 1, 1.0f};
  KGroupedTiles::Params tp{offsets, E};
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int bn = Kw % 256 == 0 ? 256 : 128;
  const int tiles = E * (Nw / 128) * (Kw / bn);
  // GEMM: M = Nw (A = dY MN-major [rows][Nw]), N = Kw (B = X MN-major [rows][Kw]), K = rows
  if (bn == 256)
    return launch_gemm_inst<256, true, true, StoreEpi, KGroupedTiles>(dY, X, Nw, Kw, max_rows, lddy, ldx, ep, status, s, 0,
                                                                       1, tp, max_rows, max_rows, tiles);
  return launch_gemm_inst<128, true, true, StoreEpi, KGroupedTiles>(dY, X, Nw, Kw, max_rows, lddy, ldx, ep, status, s, 0, 1,
                                                                     tp, max_rows, max_rows, tiles);
}

// ------------------------------------------------------------------ tensor-parallel fused GEMMs
// All-gather -> GEMM: Y[T][N] = concat_r(X_r)[T][K] * op(W), X_r = rank r's [rows_per_rank][K] shard in
// symmetric memory (x_ptrs[r] = its address mapped into this process). T = world * rows_per_rank,
// rows_per_rank % 128 == 0. b_mn = 0: W is [N][K] (forward); b_mn = 1: W is [K][N] (dgrad through a
// row-parallel layer). The caller has made sure (device barrier) that every rank's shard is complete.
extern "C" int axb_gemm_allgather_a(const unsigned long long* x_ptrs, int world, int rank, const void* W, void* Y,
                                    int rows_per_rank, int N, int K, long long ldx, long long ldw, long long ldy,
                                    int b_mn, int out_fp32, int* status, void* stream) {
  using namespace axb;
  if (world < 1 || world > PeerGatherTiles::MAX_RANKS || rank < 0 || rank >= world || rows_per_rank <= 0 ||
      rows_per_rank % GEMM_BM != 0 || (ldx & 7) || (ldw & 7))
    return AXB_LAUNCH_BAD_ARG;
  PeerGatherTiles::Params tp;
  for (int r = 0; r < PeerGatherTiles::MAX_RANKS; ++r) {
    const void* base = reinterpret_cast<const void*>(x_ptrs[r < world ? r : rank]);
    int rc = make_tmap_2d(&tp.maps[r], base, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, rows_per_rank, ldx * 2, GEMM_BK,
                          GEMM_BM, true);
    if (rc != AXB_LAUNCH_OK) return rc;
  }
  tp.world = world;
  tp.rank = rank;
  tp.blocks_per_rank = rows_per_rank / GEMM_BM;
  const int T = world * rows_per_rank;
  StoreEpi::Params ep{Y, ldy, out_fp32 ? 1 : 0, 1.0f};
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const void* own = reinterpret_cast<const void*>(x_ptrs[rank]);
  const int bn = (N % 256 == 0 || N > 2048) ? 256 : 128;
#define AXB_AG(BN_, BMN_)                                                                                     \
  return launch_gemm_inst<BN_, false, BMN_, StoreEpi, PeerGatherTiles>(own, W, T, N, K, ldx, ldw, ep, status, s, 0, 1, tp, \
                                                                      rows_per_rank, -1)
  if (bn == 256) {
    if (b_mn) AXB_AG(256, true);
    AXB_AG(256, false);
  }
  if (b_mn) AXB_AG(128, true);
  AXB_AG(128, false);
#undef AXB_AG
}

// Weight all-gather fused into the consuming GEMM (ZeRO-3 / FSDP style parameter sharding):
//   Y[T][F] = X[T][K] * concat_r(W_r)^T,  W_r = rank r's row shard [F / world][K] in peer-visible memory.
// The weights ride on the 128-row side of the MMA (each weight tile is fetched by TMA through the tensor map
// of the rank that owns it, own shard first), the tokens on the N side, and the epilogue stores transposed,
// so no gathered copy of W is ever materialised. feats_per_rank must be a multiple of 128.
extern "C" int axb_gemm_gather_weights(const unsigned long long* w_ptrs, int world, int rank, const void* X, void* Y,
                                       int feats_per_rank, int T, int K, long long ldw, long long ldx, long long ldy,
                                       int out_fp32, int* status, void* stream) {
  using namespace axb;
  if (world < 1 || world > PeerGatherTiles::MAX_RANKS || rank < 0 || rank >= world || feats_per_rank <= 0 ||
      feats_per_rank % GEMM_BM != 0 || T <= 0 || (ldx & 7) || (ldw & 7))
    return AXB_LAUNCH_BAD_ARG;
  PeerGatherTiles::Params tp;
  for (int r = 0; r < PeerGatherTiles::MAX_RANKS; ++r) {
    const void* base = reinterpret_cast<const void*>(w_ptrs[r < world ? r : rank]);
    int rc = make_tmap_2d(&tp.maps[r], base, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, feats_per_rank, ldw * 2, GEMM_BK,
                          GEMM_BM, true);
    if (rc != AXB_LAUNCH_OK) return rc;
  }
  tp.world = world;
  tp.rank = rank;
  tp.blocks_per_rank = feats_per_rank / GEMM_BM;
  const int F = world * feats_per_rank;
  TransposedEpi::Params ep{Y, ldy, out_fp32 ? 1 : 0, nullptr};
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const void* own = reinterpret_cast<const void*>(w_ptrs[rank]);
  if (T % 256 == 0 || T > 2048)
    return launch_gemm_inst<256, false, false, TransposedEpi, PeerGatherTiles>(own, X, F, T, K, ldw, ldx, ep, status, s, 0, 1, tp,
                                                                                feats_per_rank, -1);
  return launch_gemm_inst<128, false, false, TransposedEpi, PeerGatherTiles>(own, X, F, T, K, ldw, ldx, ep, status, s, 0, 1, tp,
                                                                              feats_per_rank, -1);
}

// GEMM -> reduce-scatter, part 1: partial[T][N] = X[T][K] * op(W); the epilogue stores every tile into the
// staging slot [rank][local row][N] of the rank that owns the rows (staging_ptrs[r], bf16, row pitch ld).
extern "C" int axb_gemm_scatter(const void* X, const void* W, const unsigned long long* staging_ptrs, int world, int rank,
                                int T, int N, int K, long long ldx, long long ldw, long long ld, int b_mn, int* status,
                                void* stream) {
  using namespace axb;
  if (world < 1 || world > PeerScatterEpi::MAX_RANKS || rank < 0 || rank >= world || T <= 0 || T % world != 0 ||
      (ldx & 7) || (ldw & 7))
    return AXB_LAUNCH_BAD_ARG;
  PeerScatterEpi::Params ep;
  for (int r = 0; r < PeerScatterEpi::MAX_RANKS; ++r) ep.staging[r] = reinterpret_cast<void*>(staging_ptrs[r < world ? r : rank]);
  ep.ld = ld;
  ep.rows_per_rank = T / world;
  ep.rank = rank;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int bn = (N % 256 == 0 || N > 2048) ? 256 : 128;
  if (bn == 256) {
    if (b_mn) return launch_gemm_inst<256, false, true, PeerScatterEpi>(X, W, T, N, K, ldx, ldw, ep, status, s, 0);
    return launch_gemm_inst<256, false, false, PeerScatterEpi>(X, W, T, N, K, ldx, ldw, ep, status, s, 0);
  }
  if (b_mn) return launch_gemm_inst<128, false, true, PeerScatterEpi>(X, W, T, N, K, ldx, ldw, ep, status, s, 0);
  return launch_gemm_inst<128, false, false, PeerScatterEpi>(X, W, T, N, K, ldx, ldw, ep, status, s, 0);
}

namespace axb {
// out[r][c] = sum over source ranks (in rank order) of staging[src][r][c] (+ residual), bf16 in / out.
__global__ void rs_reduce_kernel(const __nv_bfloat16* __restrict__ staging, const __nv_bfloat16* __restrict__ residual,
                                 __nv_bfloat16* __restrict__ out, int world, long long rows, int N, long long ld,
                                 long long ldo) {
  const long long vec_per_row = N / 8;
  const long long total = rows * vec_per_row;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / vec_per_row, v = i - r * vec_per_row;
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int s = 0; s < world; ++s) {
      const uint4 q = reinterpret_cast<const uint4*>(staging + (static_cast<long long>(s) * rows + r) * ld)[v];
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(h[j]);
        acc[2 * j] += f.x;
        acc[2 * j + 1] += f.y;
      }
    }
    if (residual != nullptr) {
      const uint4 q = reinterpret_cast<const uint4*>(residual + r * ldo)[v];
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(h[j]);
        acc[2 * j] += f.x;
        acc[2 * j + 1] += f.y;
      }
    }
    uint4 o;
    o.x = pack_bf16x2(acc[0], acc[1]);
    o.y = pack_bf16x2(acc[2], acc[3]);
    o.z = pack_bf16x2(acc[4], acc[5]);
    o.w = pack_bf16x2(acc[6], acc[7]);
    reinterpret_cast<uint4*>(out + r * ldo)[v] = o;
  }
}
}  // namespace axb

// GEMM -> reduce-scatter, part 2 (after a barrier): sum this rank's staging slots in rank order.
extern "C" int axb_rs_reduce(const void* staging, const void* residual, void* out, int world, long long rows, int N,
                             long long ld, long long ldo, void* stream) {
  using namespace axb;
  if (world < 1 || rows <= 0 || N % 8 != 0 || (ld & 7) || (ldo & 7)) return AXB_LAUNCH_BAD_ARG;
  const long long total = rows * (N / 8);
  long long blocks = (total + 255) / 256;
  const long long cap = static_cast<long long>(sm_count()) * 8;
  if (blocks > cap) blocks = cap;
  rs_reduce_kernel<<<static_cast<int>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(staging), static_cast<const __nv_bfloat16*>(residual),
      static_cast<__nv_bfloat16*>(out), world, rows, N, ld, ldo);
  return check_launch();
}

// ------------------------------------------------------------------------- lightning indexer
// logits[s][j] = sum_h w[s][h] * relu(q[s][h] . k[j]) inside the window [ks[s], ke[s]), -inf outside.
// The product runs as one GEMM with the KEYS on the 128-row side and the (query, head) pairs as columns, so an
// epilogue thread (one accumulator row = one key) holds 32 consecutive heads of one query in its registers:
// ReLU, head weight and the sum over heads are 32 fused multiply-adds on the accumulator, no shuffles, and
// the 32 lanes of a warp then write 32 consecutive logits of that query. With 64 / 128 / 256 heads the
// partial sums of consecutive 32-column chunks are carried in a register (a tile is 128 / 256 columns wide,
// so a query never straddles tiles); the result is bit-reproducible.
namespace axb {
struct IndexerEpi {
  struct Params {
    float* logits;     // [S][ld]
    long long ld;
    const float* w;    // [S * heads]
    const int* ks;
    const int* ke;
    int heads;
  };
  const Params& p;
  const GemmShape& sh;
  int row;             // key index
  float carry;
  // head weights and window of the NEXT chunk, loaded one chunk ahead: the epilogue visits a tile's chunks one
  // after another with a tensor-memory load in between, so a load issued here has that long to arrive
  float4 wn[8];
  int ks_n, ke_n;
  __device__ __forceinline__ void prefetch(int col0) {
    if (col0 >= sh.N) return;
    const float4* wv = reinterpret_cast<const float4*>(p.w + col0);
#pragma unroll
    for (int j = 0; j < 8; ++j) wn[j] = wv[j];
    const int s = col0 / p.heads;
    ks_n = p.ks[s];
    ke_n = p.ke[s];
  }
  __device__ IndexerEpi(const Params& p_, int, int n_blk, int row_, const GemmShape& sh_, int)
      : p(p_), sh(sh_), row(row_), carry(0.0f), ks_n(0), ke_n(0) {
    prefetch(n_blk * tile_cols());
  }
  __device__ __forceinline__ int tile_cols() const { return (p.heads == 256 || sh.N >= 256) ? 256 : 128; }
  __device__ __forceinline__ void chunk(int col0, const uint32_t (&acc)[32]) {
    if (col0 >= sh.N) return;                       // columns = (s, h); N = S * heads is a multiple of 32
    float s0 = 0.0f, s1 = 0.0f, s2 = 0.0f, s3 = 0.0f;      // four chains: the adds of one chain wait on each other
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      s0 = fmaf(fmaxf(__uint_as_float(acc[4 * j + 0]), 0.0f), wn[j].x, s0);
      s1 = fmaf(fmaxf(__uint_as_float(acc[4 * j + 1]), 0.0f), wn[j].y, s1);
      s2 = fmaf(fmaxf(__uint_as_float(acc[4 * j + 2]), 0.0f), wn[j].z, s2);
      s3 = fmaf(fmaxf(__uint_as_float(acc[4 * j + 3]), 0.0f), wn[j].w, s3);
    }
    float sum = (s0 + s1) + (s2 + s3);
    const int lo = ks_n, hi = ke_n;
    const int s = col0 >> (31 - __clz(p.heads));           // heads is a power of two
    const int h0 = col0 - s * p.heads;
    if (((col0 + 32) & (tile_cols() - 1)) != 0) prefetch(col0 + 32);      // not past the end of this tile
    sum += (h0 == 0) ? 0.0f : carry;
    carry = sum;
    if (h0 + 32 < p.heads || row >= sh.M) return;
    p.logits[(long long)s * p.ld + row] = (row >= lo && row < hi) ? sum : -INFINITY;
  }
  __device__ __forceinline__ void finish() {}
};
}  // namespace axb

// q: bf16 [S * heads][ldq] (row = (s, h)), k: bf16 [Skv][ldk], w: fp32 [S * heads] (16-byte aligned),
// logits: fp32 [S][ld] (every element written). heads in {32, 64, 128, 256}, D % 64 == 0.
extern "C" int axb_indexer_fwd(const void* q, const void* k, const float* w, const int* ks, const int* ke, float* logits,
                               int S, int heads, int Skv, int D, long long ldq, long long ldk, long long ld, int* status,
                               void* stream) {
  using namespace axb;
  if (S <= 0 || Skv <= 0 || (heads != 32 && heads != 64 && heads != 128 && heads != 256) || D <= 0 || D % GEMM_BK != 0 ||
      (ldq & 7) || (ldk & 7) || (reinterpret_cast<uintptr_t>(w) & 15))
    return AXB_LAUNCH_BAD_ARG;
  IndexerEpi::Params ep{logits, ld, w, ks, ke, heads};
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const long long N = (long long)S * heads;
  if (N > 0x7fffffffLL) return AXB_LAUNCH_BAD_ARG;
  if (heads == 256 || N >= 256)       // a tile must hold whole queries: 256 columns unless the whole problem is narrower
    return launch_gemm_inst<256, false, false, IndexerEpi>(k, q, Skv, (int)N, D, ldk, ldq, ep, status, st, 0);
  return launch_gemm_inst<128, false, false, IndexerEpi>(k, q, Skv, (int)N, D, ldk, ldq, ep, status, st, 0);
}
