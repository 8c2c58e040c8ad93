// Small-token-batch ("decode") GEMM: out[tokens][feats] = X[tokens][K] * W[feats][K]^T.
//
// With a few hundred tokens the product has too few 128-feature output tiles to occupy 148 SMs, so
// K is split across the CTAs of a thread-block cluster: the S CTAs of a cluster work on the same
// output tile, each streaming 1/S of the weight columns through the tcgen05 pipeline into its own
// TMEM accumulator. The partial tiles never touch global memory: after the main loop each CTA
// scatters its accumulator, 32 token-columns at a time, into the shared memory of the CTA that owns
// that column group (distributed shared memory), a cluster barrier publishes the writes, and every
// CTA sums the S partials of the groups it owns in split order (deterministic) and writes the
// final bf16 / fp32 values. Weights ride on the 128-row MMA side ("swap-AB"), tokens on N.
//
// Warps: 0 = TMA producer, 1 = MMA issuer + TMEM owner, 2-5 = epilogue (TMEM lane quarters).
// Every mbarrier wait is bounded; on a timeout the CTA records an error, keeps taking part in the
// two cluster barriers (so its peers never wait for it) and the caller sees the status word.
#include "gemm_core.cuh"
#include "host_utils.h"

namespace axb {

#ifdef AXB_TIMELINE
// Development aid (compiled only with -DAXB_TIMELINE): per-CTA timestamps of the kernel's phases.
__device__ unsigned long long* g_timeline = nullptr;
__device__ __forceinline__ void tl_mark(int slot) {
  if (g_timeline != nullptr) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    g_timeline[(blockIdx.y * gridDim.x + blockIdx.x) * 8 + slot] = t;
  }
}
#define AXB_TL(slot, cond) do { if (cond) tl_mark(slot); } while (0)
#else
#define AXB_TL(slot, cond) do { } while (0)
#endif

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t cluster_nctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire;" ::: "memory");
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t local_smem_addr, uint32_t cta) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_smem_addr), "r"(cta));
  return r;
}
__device__ __forceinline__ void st_cluster_v4(uint32_t addr, float a, float b, float c, float d) {
  asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "f"(a), "f"(b), "f"(c),
               "f"(d)
               : "memory");
}

// Exchange buffer (reuses the pipeline stages once the main loop is over):
//   xbuf[src split][owned group][row 0..127][32 floats], the 16-byte quads of a row XOR-swizzled with
//   (row & 7) so that both the row-per-lane writes and reads are bank-conflict free.
template <int BN>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_decode_cluster_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX,
                           int feats, int tokens, int K, void* __restrict__ out, long long ldc,
                           int out_fp32, int* status) {
  using S = GemmSmem<BN>;
  constexpr int NCHUNK = BN / 32;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + S::STAGES * S::STAGE_BYTES);
  uint64_t* full = bars;
  uint64_t* empty = bars + S::STAGES;
  uint64_t* acc_full = bars + 2 * S::STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_full + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  AXB_TL(0, threadIdx.x == 0);
  const int split = static_cast<int>(cluster_ctarank());
  const int csize = static_cast<int>(cluster_nctarank());
  const int num_m = (feats + GEMM_BM - 1) / GEMM_BM;
  const int m_blk = blockIdx.y % num_m;
  const int n_blk = blockIdx.y / num_m;
  const int num_k = (K + GEMM_BK - 1) / GEMM_BK;
  const int k_per = (num_k + csize - 1) / csize;
  const int kb0 = split * k_per;
  const int kb1 = min(num_k, kb0 + k_per);
  const bool has_work = kb0 < kb1;
  const int max_own = (NCHUNK + csize - 1) / csize;
  // the exchange buffer (csize x max_own slots of 16 KB) must fit in the pipeline stages
  const bool fits = csize * max_own * (GEMM_BM * 128) <= S::STAGES * S::STAGE_BYTES;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S::STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(acc_full, 1);
    mbar_fence_init();
    tma_prefetch_desc(&tmW);
    tma_prefetch_desc(&tmX);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, BN);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  bool ok = true;
  AXB_TL(1, threadIdx.x == 0);

  if (warp == 0) {
    if (lane == 0) {
      int s = 0;
      uint32_t ph = 0;
      for (int kb = kb0; kb < kb1; ++kb) {
        if (!mbar_wait(&empty[s], ph ^ 1)) {
          report_error(status, AXB_ERR_WAIT_EMPTY);
          break;
        }
        uint8_t* sA = smem + s * S::STAGE_BYTES;
        mbar_expect_tx(&full[s], S::STAGE_BYTES);
        tma_load_2d(sA, &tmW, &full[s], kb * GEMM_BK, m_blk * GEMM_BM);
        tma_load_2d(sA + S::A_BYTES, &tmX, &full[s], kb * GEMM_BK, n_blk * BN);
        if (++s == S::STAGES) {
          s = 0;
          ph ^= 1;
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && has_work) {
      constexpr uint32_t idesc = umma_idesc(GEMM_BM, BN, 0u, 0u);
      int s = 0;
      uint32_t ph = 0;
      bool issued = true;
      for (int kb = kb0; kb < kb1; ++kb) {
        if (!mbar_wait(&full[s], ph)) {
          report_error(status, AXB_ERR_WAIT_FULL);
          issued = false;
          break;
        }
        tc_fence_after();
        const uint32_t a0 = smem_u32(smem + s * S::STAGE_BYTES);
        const uint32_t b0 = a0 + S::A_BYTES;
#pragma unroll
        for (int j = 0; j < GEMM_BK / 16; ++j)
          umma_f16_ss(tmem_base, umma_smem_desc(a0 + j * 32, 16, 1024), umma_smem_desc(b0 + j * 32, 16, 1024),
                      idesc, (kb != kb0 || j != 0) ? 1u : 0u);
        tc_commit(&empty[s]);
        if (++s == S::STAGES) {
          s = 0;
          ph ^= 1;
        }
      }
      if (issued) tc_commit(acc_full);
      AXB_TL(2, true);
    }
  } else {
    // The accumulator is complete (and with it every read of this CTA's pipeline stages) once
    // acc_full fires; only then may peers overwrite the stages with their partial tiles.
    if (has_work && !mbar_wait(acc_full, 0)) {
      report_error(status, AXB_ERR_WAIT_TMEM_FULL);
      ok = false;
    }
    tc_fence_after();
    AXB_TL(3, threadIdx.x == 64);
  }

  __syncwarp();
  cluster_sync_all();   // #1: every CTA of the cluster is done with its stages
  AXB_TL(4, threadIdx.x == 64);

  const uint32_t xbuf = smem_u32(smem);
  if (!fits) {
    if (threadIdx.x == 0) report_error(status, AXB_ERR_BAD_ARG);
  } else if (warp >= 2) {
    tc_fence_after();
    const int q = warp & 3;
    const int row = q * 32 + lane;   // feature row inside the tile
    const uint32_t t0 = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
#pragma unroll 1
    for (int c = 0; c < NCHUNK; ++c) {
      uint32_t acc[32];
      if (has_work && ok) {
        tmem_ld_32x32(t0 + c * 32, acc);
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) acc[j] = 0u;
      }
      const int owner = c % csize;
      const int oi = c / csize;
      const uint32_t local = xbuf + static_cast<uint32_t>(((split * max_own + oi) * GEMM_BM + row) * 128);
      const uint32_t remote = map_to_cta(local, static_cast<uint32_t>(owner));
#pragma unroll
      for (int g = 0; g < 8; ++g)
        st_cluster_v4(remote + static_cast<uint32_t>(((g ^ (row & 7)) << 4)), __uint_as_float(acc[4 * g]),
                      __uint_as_float(acc[4 * g + 1]), __uint_as_float(acc[4 * g + 2]),
                      __uint_as_float(acc[4 * g + 3]));
    }
    tc_fence_before();
  }

  AXB_TL(5, threadIdx.x == 64);
  __syncwarp();
  cluster_sync_all();   // #2: all partial tiles have landed
  AXB_TL(6, threadIdx.x == 64);

  if (warp >= 2 && fits) {
    const int q = warp & 3;
    const int row = q * 32 + lane;
    const int f = m_blk * GEMM_BM + row;
#pragma unroll 1
    for (int oi = 0; oi < max_own; ++oi) {
      const int c = oi * csize + split;
      if (c >= NCHUNK) break;
      float sum[32];
#pragma unroll
      for (int j = 0; j < 32; ++j) sum[j] = 0.f;
      for (int s = 0; s < csize; ++s) {
        const uint8_t* base = smem + ((s * max_own + oi) * GEMM_BM + row) * 128;
#pragma unroll
        for (int g = 0; g < 8; ++g) {
          const float4 v = *reinterpret_cast<const float4*>(base + ((g ^ (row & 7)) << 4));
          sum[4 * g] += v.x;
          sum[4 * g + 1] += v.y;
          sum[4 * g + 2] += v.z;
          sum[4 * g + 3] += v.w;
        }
      }
      const int tok0 = n_blk * BN + c * 32;
      if (f < feats) {
        if (out_fp32) {
          float* o = reinterpret_cast<float*>(out) + static_cast<long long>(tok0) * ldc + f;
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (tok0 + j < tokens) o[static_cast<long long>(j) * ldc] = sum[j];
        } else {
          __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(out) + static_cast<long long>(tok0) * ldc + f;
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (tok0 + j < tokens) o[static_cast<long long>(j) * ldc] = __float2bfloat16(sum[j]);
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  AXB_TL(7, threadIdx.x == 0);
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, BN);
  }
}

template <int BN>
static int launch_decode(const void* X, const void* W, void* out, int tokens, int feats, int K, long long ldx,
                         long long ldw, long long ldc, int out_fp32, int csize, int* status, cudaStream_t stream) {
  CUtensorMap tmW, tmX;
  int rc = make_tmap_2d(&tmW, W, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, feats, ldw * 2, GEMM_BK, GEMM_BM, true);
  if (rc != AXB_LAUNCH_OK) return rc;
  rc = make_tmap_2d(&tmX, X, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, tokens, ldx * 2, GEMM_BK, BN, true);
  if (rc != AXB_LAUNCH_OK) return rc;
  auto kern = gemm_decode_cluster_kernel<BN>;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, GemmSmem<BN>::TOTAL) != cudaSuccess)
      return AXB_LAUNCH_CUDA_ERROR;
    attr_set = true;
  }
  const int tiles = ((feats + GEMM_BM - 1) / GEMM_BM) * ((tokens + BN - 1) / BN);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(csize, tiles, 1);
  cfg.blockDim = dim3(GEMM_THREADS, 1, 1);
  cfg.dynamicSmemBytes = GemmSmem<BN>::TOTAL;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = csize;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (cudaLaunchKernelEx(&cfg, kern, tmW, tmX, feats, tokens, K, out, ldc, out_fp32, status) != cudaSuccess) {
    cudaGetLastError();
    return AXB_LAUNCH_CUDA_ERROR;
  }
  return check_launch();
}

}  // namespace axb

#ifdef AXB_TIMELINE
extern "C" int axb_gemm_decode_set_timeline(unsigned long long* buf) {
  return cudaMemcpyToSymbol(axb::g_timeline, &buf, sizeof(buf)) == cudaSuccess ? 0 : -4;
}
#endif

static int g_forced_cluster = 0;
// Experiments only: force the cluster size of the next launches (0 restores the heuristic).
extern "C" void axb_gemm_decode_force_cluster(int cs) { g_forced_cluster = cs; }

// Cluster size (= K splits) the cluster kernel would use for this shape, or 0 when the shape is
// better served by the persistent kernel (enough output tiles to fill the GPU on their own).
extern "C" int axb_gemm_decode_max_active_clusters(int bn, int csize);

extern "C" int axb_gemm_decode_cluster_size(int tokens, int feats, int K) {
  using namespace axb;
  const int bn = tokens <= 64 ? 64 : (tokens <= 128 ? 128 : 256);
  const int tiles = ((feats + GEMM_BM - 1) / GEMM_BM) * ((tokens + bn - 1) / bn);
  const int num_k = (K + GEMM_BK - 1) / GEMM_BK;
  const int sms = sm_count();
  if (tiles * 2 > sms) return 0;
  int s = sms / tiles;
  if (s > 8) s = 8;
  while (s > 1 && num_k / s < 4) --s;   // at least four K blocks per CTA
  // every split must own at least one K block (k_per = ceil(num_k / s))
  while (s > 1 && (s - 1) * ((num_k + s - 1) / s) >= num_k) --s;
  // exchange buffer: s * ceil(chunks / s) slots of 16 KB must fit in the 192 KB of pipeline stages
  const int chunks = bn / 32;
  while (s > 1 && s * ((chunks + s - 1) / s) > 12) --s;
  // one wave: a cluster lives inside one GPC, so fewer clusters fit than sms / s suggests
  static int fit[3][9];
  static bool have[3][9];
  const int bi = bn == 64 ? 0 : (bn == 128 ? 1 : 2);
  while (s > 1) {
    if (!have[bi][s]) {
      fit[bi][s] = axb_gemm_decode_max_active_clusters(bn, s);
      have[bi][s] = true;
    }
    if (fit[bi][s] < 0 || fit[bi][s] >= tiles) break;
    --s;
  }
  return s < 2 ? 0 : s;
}

// Diagnostics: how many clusters of `csize` CTAs of the BN-wide kernel the device can hold at once.
extern "C" int axb_gemm_decode_max_active_clusters(int bn, int csize) {
  using namespace axb;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(csize, 64, 1);
  cfg.blockDim = dim3(GEMM_THREADS, 1, 1);
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = csize;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int n = -1;
  cudaError_t e;
  if (bn == 64) {
    cfg.dynamicSmemBytes = GemmSmem<64>::TOTAL;
    cudaFuncSetAttribute(gemm_decode_cluster_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, GemmSmem<64>::TOTAL);
    e = cudaOccupancyMaxActiveClusters(&n, gemm_decode_cluster_kernel<64>, &cfg);
  } else if (bn == 128) {
    cfg.dynamicSmemBytes = GemmSmem<128>::TOTAL;
    cudaFuncSetAttribute(gemm_decode_cluster_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, GemmSmem<128>::TOTAL);
    e = cudaOccupancyMaxActiveClusters(&n, gemm_decode_cluster_kernel<128>, &cfg);
  } else {
    cfg.dynamicSmemBytes = GemmSmem<256>::TOTAL;
    cudaFuncSetAttribute(gemm_decode_cluster_kernel<256>, cudaFuncAttributeMaxDynamicSharedMemorySize, GemmSmem<256>::TOTAL);
    e = cudaOccupancyMaxActiveClusters(&n, gemm_decode_cluster_kernel<256>, &cfg);
  }
  if (e != cudaSuccess) {
    cudaGetLastError();
    return -1;
  }
  return n;
}

// out[tokens][ldc] = X[tokens][ldx] * W[feats][ldw]^T, bf16 inputs, bf16 or fp32 output.
// Returns AXB_LAUNCH_BAD_ARG when the shape does not qualify (see axb_gemm_decode_cluster_size).
extern "C" int axb_gemm_decode_cluster(const void* X, const void* W, void* out, int tokens, int feats, int K,
                                       long long ldx, long long ldw, long long ldc, int out_fp32, int* status,
                                       void* stream) {
  using namespace axb;
  if (tokens <= 0 || feats <= 0 || K <= 0 || (ldx & 7) || (ldw & 7)) return AXB_LAUNCH_BAD_ARG;
  int cs = axb_gemm_decode_cluster_size(tokens, feats, K);
  if (g_forced_cluster > 0) cs = g_forced_cluster;
  if (cs < 2) return AXB_LAUNCH_BAD_ARG;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (tokens <= 64) return launch_decode<64>(X, W, out, tokens, feats, K, ldx, ldw, ldc, out_fp32, cs, status, s);
  if (tokens <= 128) return launch_decode<128>(X, W, out, tokens, feats, K, ldx, ldw, ldc, out_fp32, cs, status, s);
  return launch_decode<256>(X, W, out, tokens, feats, K, ldx, ldw, ldc, out_fp32, cs, status, s);
}
