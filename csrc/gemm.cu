// extern "C" launchers for the plain bf16 GEMM built on gemm_core.cuh.
#include "gemm_core.cuh"
#include "host_utils.h"

namespace axb {

template <int BN, bool A_MN, bool B_MN, class Epi>
static int launch_gemm_inst(const void* A, const void* B, int M, int N, int K, long long lda,
                            long long ldb, const typename Epi::Params& ep, int* status,
                            cudaStream_t stream, int max_ctas) {
  CUtensorMap tmA, tmB;
  int rc;
  if (!A_MN)
    rc = make_tmap_2d(&tmA, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, M, lda * 2, GEMM_BK, GEMM_BM, true);
  else
    rc = make_tmap_2d(&tmA, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, M, K, lda * 2, 64, GEMM_BK, true);
  if (rc != AXB_LAUNCH_OK) return rc;
  if (!B_MN)
    rc = make_tmap_2d(&tmB, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, N, ldb * 2, GEMM_BK, BN, true);
  else
    rc = make_tmap_2d(&tmB, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, N, K, ldb * 2, 64, GEMM_BK, true);
  if (rc != AXB_LAUNCH_OK) return rc;

  auto kern = gemm_tc_kernel<BN, A_MN, B_MN, Epi>;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             GemmSmem<BN>::TOTAL) != cudaSuccess)
      return AXB_LAUNCH_CUDA_ERROR;
    attr_set = true;
  }
  const int num_tiles = ((M + GEMM_BM - 1) / GEMM_BM) * ((N + BN - 1) / BN);
  int grid = sm_count();
  if (max_ctas > 0 && max_ctas < grid) grid = max_ctas;
  if (num_tiles < grid) grid = num_tiles;
  GemmShape sh{M, N, K};
  kern<<<grid, GEMM_THREADS, GemmSmem<BN>::TOTAL, stream>>>(tmA, tmB, sh, ep, status);
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
