// Paged decode attention for batches whose sequences share a prefix (the n samples of one prompt).
//
// The pages of a shared prompt are the same physical pages in every sample's block table, and the plain
// decode kernel streams them once per sample: n times the tensor work and n times the per-tile latency
// chain for identical keys. Here attention over a batch is a list of ITEMS, each one CTA group:
//   * a prefix item per group of samples: the queries of up to 32 / rep sequences (rep = query heads per
//     KV head) ride together as the N dimension of the transposed products
//         S^T[128 keys x 32] = K_tile * Q^T      O^T[128 dims x 32] += V_tile^T * P^T
//     over the group's shared pages, so every shared K/V tile is fetched and multiplied once per group;
//   * a suffix item per sequence over its own pages (from its first private page on).
// Every item writes un-normalised partial results (max, sum, O) into per-(sequence, head) slots; the
// merge kernel of the plain path combines a sequence's suffix splits and its prefix slot. A sequence
// without a shared prefix gets neutral prefix slots from its suffix item.
//
// Same tile pipeline as paged_decode_kernel (3-stage TMA ring of 64 KB K|V page tiles, tcgen05 products,
// thread t owns key t for the softmax and output dimension t in the epilogue; the running maximum is raised
// lazily); waits are bounded.
#include "ptx.cuh"
#include "host_utils.h"

namespace axb {

constexpr int PS_D = 128;
constexpr int PS_PAGE = 128;
constexpr int PS_TILE = PS_PAGE * PS_D * 2;  // 32 KB
constexpr int PS_STAGES = 3;

__device__ __forceinline__ uint32_t ps_sw128(int row, int col_elem) {
  const int unit = (col_elem >> 3) ^ (row & 7);
  return row * 128 + unit * 16 + (col_elem & 7) * 2;
}

template <int NCOL>
struct PsCfg {
  static constexpr int NPAD = NCOL <= 16 ? 16 : 32;                 // MMA N
  static constexpr int QBYTES = 2 * NPAD * 128;                      // [2 K-chunks][NPAD rows][64] bf16
  static constexpr int SMEM = PS_STAGES * 2 * PS_TILE + 2 * QBYTES + 2 * 4 * NCOL * 4 + 256 + 1024;
};

// items: first[w] (batch index of the item's first sequence), size[w] (sequences, 0 = inactive), page0[w]
// (first page column of the block table row of `first`), keys[w] (keys from that page on), slot[w] (first
// partial slot the item's splits write). nslots = partial slots per (sequence, head).
// neutral_from / neutral_n: when neutral_n > 0 and page0 == 0, the item also neutralises slots
// [neutral_from, neutral_from + neutral_n) of its sequences (no shared prefix exists for them).
template <int NCOL>
__global__ void __launch_bounds__(128, 1)
paged_decode_items_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                          const __nv_bfloat16* __restrict__ q, long long q_row_stride,
                          const int* __restrict__ block_table, int max_pages, const int* __restrict__ item_first,
                          const int* __restrict__ item_size, const int* __restrict__ item_page0,
                          const int* __restrict__ item_keys, int slot0, int neutral_from, int neutral_n,
                          float* __restrict__ part_o, float* __restrict__ part_ml, int Hq, int Hkv, int nsplit,
                          int nslots, float scale_log2, int* status) {
  using Cfg = PsCfg<NCOL>;
  constexpr int NPAD = Cfg::NPAD;
  grid_launch_dependents();
  const int hk = blockIdx.x, w = blockIdx.y, sp = blockIdx.z;
  const int rep = Hq / Hkv;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int gsize = item_size[w];
  if (gsize <= 0) return;
  const int b0 = item_first[w];
  const int page0 = item_page0[w];
  const int n_keys = item_keys[w];
  const int ncols = min(gsize * rep, NCOL);
  const int n_blocks = (n_keys + PS_PAGE - 1) / PS_PAGE;
  const int per = (n_blocks + nsplit - 1) / nsplit;
  const int blk_begin = sp * per;
  const int blk_end = min(n_blocks, blk_begin + per);
  const int nb = blk_end - blk_begin;

  // slots this item never fills for its sequences: no shared prefix -> neutral prefix slots
  if (neutral_n > 0 && page0 == 0 && sp == 0) {
    for (int i = tid; i < ncols * neutral_n; i += 128) {
      const int c = i / neutral_n, sl = i % neutral_n;
      const long long idx = ((long long)(b0 + c / rep) * Hq + hk * rep + c % rep) * nslots + neutral_from + sl;
      part_ml[idx * 2] = -1e30f;
      part_ml[idx * 2 + 1] = 0.f;
    }
  }
  if (nb <= 0) {
    if (tid < ncols) {
      const long long idx = ((long long)(b0 + tid / rep) * Hq + hk * rep + tid % rep) * nslots + slot0 + sp;
      part_ml[idx * 2] = -1e30f;
      part_ml[idx * 2 + 1] = 0.f;
    }
    return;
  }

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sKV = smem;                                  // [stage][K 32K | V 32K]
  uint8_t* sQ = smem + PS_STAGES * 2 * PS_TILE;         // [2 chunks][NPAD rows][64] bf16
  uint8_t* sP = sQ + Cfg::QBYTES;
  float* red = reinterpret_cast<float*>(sP + Cfg::QBYTES);   // [2][4 warps][NCOL]
  uint64_t* bars = reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(red) + 2 * 4 * NCOL * 4);
  uint64_t* full = bars;                                // [PS_STAGES]
  uint64_t* bar_mma = bars + PS_STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + PS_STAGES + 1);

  if (tid == 0) {
    for (int s = 0; s < PS_STAGES; ++s) mbar_init(&full[s], 1);
    mbar_init(bar_mma, 1);
    mbar_fence_init();
  }
  if (warp == 0) {
    tmem_alloc(tmem_slot, 2 * NPAD);
    tmem_relinquish();
  }
  // Q^T operand: row c = (sequence c / rep of the item, head c % rep of the kv group), zero padded to NPAD rows
  for (int i = tid; i < Cfg::QBYTES / 16; i += 128) reinterpret_cast<uint4*>(sQ)[i] = make_uint4(0, 0, 0, 0);
  __syncthreads();
  for (int c = 0; c < ncols; ++c) {
    const __nv_bfloat16 v = q[(long long)(b0 + c / rep) * q_row_stride + (long long)(hk * rep + c % rep) * PS_D + tid];
    *reinterpret_cast<__nv_bfloat16*>(sQ + (tid >> 6) * (NPAD * 128) + ps_sw128(c, tid & 63)) = v;
  }
  fence_async_shared();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tS = tmem_base + (static_cast<uint32_t>(warp * 32) << 16);
  const uint32_t tO = tS + NPAD;
  constexpr uint32_t idesc_s = umma_idesc(128, NPAD, 0, 0);
  constexpr uint32_t idesc_o = umma_idesc(128, NPAD, 1, 0);
  const int* bt = block_table + (long long)b0 * max_pages + page0;

  auto issue_load = [&](int i) {  // i-th block of this split -> stage i % STAGES
    const int s = i % PS_STAGES;
    const int page = bt[blk_begin + i];
    const int row0 = (page * Hkv + hk) * PS_PAGE;
    uint8_t* k = sKV + s * 2 * PS_TILE;
    mbar_expect_tx(&full[s], 2 * PS_TILE);
    tma_load_2d(k, &tmK, &full[s], 0, row0);
    tma_load_2d(k + 16384, &tmK, &full[s], 64, row0);
    tma_load_2d(k + PS_TILE, &tmV, &full[s], 0, row0);
    tma_load_2d(k + PS_TILE + 16384, &tmV, &full[s], 64, row0);
  };
  if (tid == 0) {
    for (int i = 0; i < PS_STAGES - 1 && i < nb; ++i) issue_load(i);
  }

  float m_run[NCOL], l_thr[NCOL];
#pragma unroll
  for (int c = 0; c < NCOL; ++c) {
    m_run[c] = -1e30f;
    l_thr[c] = 0.f;
  }
  bool ok = true;
  uint32_t ph = 0;  // bar_mma completes once per block (after S) and once after the last P*V
  for (int i = 0; i < nb; ++i) {
    const int s = i % PS_STAGES;
    const uint32_t kaddr = smem_u32(sKV + s * 2 * PS_TILE);
    if (tid == 0 && ok) {
      if (!mbar_wait(&full[s], (i / PS_STAGES) & 1)) {
        report_error(status, AXB_ERR_WAIT_FULL);
        ok = false;
      }
      tc_fence_after();
      const uint32_t qaddr = smem_u32(sQ);
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        umma_f16_ss(tmem_base, umma_smem_desc(kaddr + (ks >> 2) * 16384 + (ks & 3) * 32, 16, 1024),
                    umma_smem_desc(qaddr + (ks >> 2) * (NPAD * 128) + (ks & 3) * 32, 16, 1024), idesc_s, ks != 0);
      }
      tc_commit(bar_mma);  // also covers the P*V product of the previous block
    }
    __syncwarp();
    if (ok && !mbar_wait(bar_mma, ph)) {
      report_error(status, AXB_ERR_WAIT_TMEM_FULL);
      ok = false;
    }
    ph ^= 1;
    tc_fence_after();
    // the stage of block i-1 is free now: prefetch block i + STAGES - 1 into it
    if (tid == 0 && ok && i + PS_STAGES - 1 < nb) issue_load(i + PS_STAGES - 1);

    uint32_t sv[NPAD];
    tmem_ld_32x16(tS, sv);
    if (NPAD == 32) tmem_ld_32x16(tS + 16, sv + 16);
    tmem_ld_wait();
    const int kpos = (blk_begin + i) * PS_PAGE + tid;
    const bool valid = kpos < n_keys;
    float sc[NCOL];
#pragma unroll
    for (int c = 0; c < NCOL; ++c) {
      sc[c] = (valid && c < ncols) ? __uint_as_float(sv[c]) * scale_log2 : -INFINITY;
      const float wm = warp_max_redux(sc[c]);
      if (lane == 0) red[((i & 1) * 4 + warp) * NCOL + c] = wm;
    }
    __syncthreads();
    float alpha[NCOL];
    bool changed = false;
#pragma unroll
    for (int c = 0; c < NCOL; ++c) {
      const float* r = red + (i & 1) * 4 * NCOL + c;
      const float bm = fmaxf(fmaxf(r[0], r[NCOL]), fmaxf(r[2 * NCOL], r[3 * NCOL]));
      // the running maximum is raised only when a block exceeds it by more than 2^8: probabilities stay below
      // 256 (exact after the final normalisation) and the accumulator is rescaled on few blocks
      const bool raise = bm > m_run[c] + 8.f;
      const float mn = raise ? bm : m_run[c];
      alpha[c] = raise ? exp2f(m_run[c] - mn) : 1.f;
      changed |= raise;
      m_run[c] = mn;
      const float p = exp2f(sc[c] - mn);
      l_thr[c] = l_thr[c] * alpha[c] + p;
      if (c < ncols)
        *reinterpret_cast<__nv_bfloat16*>(sP + (tid >> 6) * (NPAD * 128) + ps_sw128(c, tid & 63)) = __float2bfloat16(p);
    }
    if (i > 0 && changed) {  // uniform across the CTA: m_run is identical in every thread
      uint32_t o[NPAD];
      tmem_ld_32x16(tO, o);
      if (NPAD == 32) tmem_ld_32x16(tO + 16, o + 16);
      tmem_ld_wait();
#pragma unroll
      for (int c = 0; c < NCOL; ++c) o[c] = __float_as_uint(__uint_as_float(o[c]) * alpha[c]);
#pragma unroll
      for (int g8 = 0; g8 < NCOL / 8; ++g8) {
        asm volatile(
            "tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
            ::"r"(tO + g8 * 8), "r"(o[g8 * 8]), "r"(o[g8 * 8 + 1]), "r"(o[g8 * 8 + 2]), "r"(o[g8 * 8 + 3]),
            "r"(o[g8 * 8 + 4]), "r"(o[g8 * 8 + 5]), "r"(o[g8 * 8 + 6]), "r"(o[g8 * 8 + 7])
            : "memory");
      }
      tmem_st_wait();
    }
    fence_async_shared();
    tc_fence_before();
    __syncthreads();
    if (tid == 0 && ok) {
      tc_fence_after();
      const uint32_t vaddr = kaddr + PS_TILE, paddr = smem_u32(sP);
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        umma_f16_ss(tmem_base + NPAD, umma_smem_desc(vaddr + ks * 2048, 16384, 1024),
                    umma_smem_desc(paddr + (ks >> 2) * (NPAD * 128) + (ks & 3) * 32, 16, 1024), idesc_o,
                    (i | ks) != 0);
      }
      if (i == nb - 1) tc_commit(bar_mma);
    }
    __syncwarp();
  }
  if (ok && !mbar_wait(bar_mma, ph)) {
    report_error(status, AXB_ERR_WAIT_TMEM_FULL);
    ok = false;
  }
  tc_fence_after();

  // ---- epilogue: un-normalised partials. l per column: reduce the per-thread sums over the CTA.
  float l_tot[NCOL];
#pragma unroll
  for (int c = 0; c < NCOL; ++c) {
    const float ws = warp_sum(l_thr[c]);
    if (lane == 0) red[warp * NCOL + c] = ws;
  }
  __syncthreads();
#pragma unroll
  for (int c = 0; c < NCOL; ++c) l_tot[c] = red[c] + red[NCOL + c] + red[2 * NCOL + c] + red[3 * NCOL + c];
  {
    uint32_t o[NPAD];
    tmem_ld_32x16(tO, o);
    if (NPAD == 32) tmem_ld_32x16(tO + 16, o + 16);
    tmem_ld_wait();
    if (ok) {
#pragma unroll
      for (int c = 0; c < NCOL; ++c) {
        if (c < ncols) {
          const long long idx = ((long long)(b0 + c / rep) * Hq + hk * rep + c % rep) * nslots + slot0 + sp;
          part_o[idx * PS_D + tid] = __uint_as_float(o[c]);
          if (tid == 0) {
            part_ml[idx * 2] = m_run[c];
            part_ml[idx * 2 + 1] = l_tot[c];
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 2 * NPAD);
  }
}

// out[b][h][:] = sum_s O_s 2^(m_s - M) / sum_s l_s 2^(m_s - M) over the nslots partial slots of (b, h)
__global__ void paged_merge_slots_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                         __nv_bfloat16* __restrict__ out, int nslots) {
  grid_launch_dependents();
  const long long bh = blockIdx.x;
  const int d = threadIdx.x;
  float M = -1e30f;
  for (int s = 0; s < nslots; ++s) M = fmaxf(M, part_ml[(bh * nslots + s) * 2]);
  float acc = 0.f, l = 0.f;
  for (int s = 0; s < nslots; ++s) {
    const float ls = part_ml[(bh * nslots + s) * 2 + 1];
    if (ls == 0.f) continue;
    const float w = exp2f(part_ml[(bh * nslots + s) * 2] - M);
    acc += part_o[(bh * nslots + s) * PS_D + d] * w;
    l += ls * w;
  }
  out[bh * PS_D + d] = __float2bfloat16(l > 0.f ? acc / l : 0.f);
}

}  // namespace axb

using namespace axb;

// Decode attention of B sequences, n_groups of which share prefixes.
//   seq_page0[b] / seq_keys[b]: first private page column and number of keys from there on (suffix item of b);
//   grp_first / grp_size / grp_keys [n_groups]: first sequence, member count (0 = inactive, at most 32 / rep)
//   and shared keys (whole pages) of every prefix item; members are consecutive sequences.
// scratch: B * Hq * (nsplit + nsplit_p) * (128 + 2) floats. The item arrays live on the device (they are
// refreshed between graph replays).
extern "C" int axb_paged_decode_shared(const void* q, long long q_row_stride, const void* kcache, const void* vcache,
                                       int num_pages, const int* block_table, int max_pages, const int* seq_first,
                                       const int* seq_one, const int* seq_page0, const int* seq_keys,
                                       const int* grp_first, const int* grp_size, const int* grp_zero,
                                       const int* grp_keys, int n_groups, void* out, int B, int Hq, int Hkv, int D,
                                       float softmax_scale, int nsplit, int nsplit_p, void* scratch, int* status,
                                       void* stream) {
  if (D != PS_D || B <= 0 || n_groups <= 0 || Hq % Hkv != 0 || Hq / Hkv > 8 || nsplit < 1 || nsplit_p < 1 || scratch == nullptr)
    return AXB_LAUNCH_BAD_ARG;
  cudaStream_t s = (cudaStream_t)stream;
  CUtensorMap tmK, tmV;
  const unsigned long long rows = (unsigned long long)num_pages * Hkv * PS_PAGE;
  int rc = make_tmap_2d(&tmK, kcache, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, PS_D, rows, PS_D * 2, 64, PS_PAGE, true);
  if (rc) return rc;
  rc = make_tmap_2d(&tmV, vcache, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, PS_D, rows, PS_D * 2, 64, PS_PAGE, true);
  if (rc) return rc;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(paged_decode_items_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, PsCfg<8>::SMEM) != cudaSuccess ||
        cudaFuncSetAttribute(paged_decode_items_kernel<32>, cudaFuncAttributeMaxDynamicSharedMemorySize, PsCfg<32>::SMEM) != cudaSuccess)
      return AXB_LAUNCH_CUDA_ERROR;
    attr_set = true;
  }
  const int nslots = nsplit + nsplit_p;
  float* part_o = reinterpret_cast<float*>(scratch);
  float* part_ml = part_o + (long long)B * Hq * nslots * PS_D;
  const float sl2 = softmax_scale * 1.4426950408889634f;
  // suffix items: one sequence each, slots [0, nsplit); they neutralise the prefix slots of unshared sequences
  paged_decode_items_kernel<8><<<dim3(Hkv, B, nsplit), 128, PsCfg<8>::SMEM, s>>>(
      tmK, tmV, (const __nv_bfloat16*)q, q_row_stride, block_table, max_pages, seq_first, seq_one, seq_page0, seq_keys,
      0, nsplit, nsplit_p, part_o, part_ml, Hq, Hkv, nsplit, nslots, sl2, status);
  rc = check_launch();
  if (rc) return rc;
  // prefix items: one group each, slots [nsplit, nsplit + nsplit_p)
  paged_decode_items_kernel<32><<<dim3(Hkv, n_groups, nsplit_p), 128, PsCfg<32>::SMEM, s>>>(
      tmK, tmV, (const __nv_bfloat16*)q, q_row_stride, block_table, max_pages, grp_first, grp_size, grp_zero, grp_keys,
      nsplit, 0, 0, part_o, part_ml, Hq, Hkv, nsplit_p, nslots, sl2, status);
  rc = check_launch();
  if (rc) return rc;
  paged_merge_slots_kernel<<<B * Hq, PS_D, 0, s>>>(part_o, part_ml, (__nv_bfloat16*)out, nslots);
  return check_launch();
}
