// Sampler-side attention over a paged KV cache (head dim 128, page = 128 tokens).
//
// Cache layout per layer: K and V are [num_pages][Hkv][128 tokens][128] bf16, so the tile of one
// (page, kv head) is a contiguous 32 KB matrix that one TMA box pair loads.
//
// Decode kernel ("swap-AB"): with one query token per sequence the natural S = q K^T has only
// Hq/Hkv useful rows, so the kernel computes the transposed products on the tensor cores instead:
//     S^T[128 keys x 16]   = K_tile[128 x 128] * Qpad^T      (A = K tile, K-major; N = heads padded to 16)
//     O^T[128 dims x 16]  += V_tile^T[128 x 128] * P^T       (A = V tile read MN-major)
// Thread t owns key t of the block for the softmax (cross-thread max per head through shared
// memory) and owns output dimension t in the epilogue. K/V tiles stream through a 3-stage TMA
// ring, so the kernel runs at the HBM rate of the cache read; the tensor work is negligible.
// Long sequences / small batches are split along the keys (grid.z) and merged by a second kernel.
//
// Replaces the FlashInfer / TRTLLM-gen paged attention that vLLM runs for the reference on
// Blackwell (axon/sampler/vllm/server.py:355-377,474-478).
#include "ptx.cuh"
#include "host_utils.h"
#include "debug.cuh"

namespace axb {

constexpr int PA_D = 128;
constexpr int PA_PAGE = 128;
constexpr int PA_TILE = PA_PAGE * PA_D * 2;  // 32 KB
constexpr int PA_STAGES = 3;
constexpr int PA_NPAD = 16;                  // query heads of one kv group, padded
constexpr int PA_SMEM = PA_STAGES * 2 * PA_TILE + 4096 /*Q*/ + 4096 /*P*/ + 1024 /*red*/ + 256 + 1024;

__device__ __forceinline__ uint32_t pa_sw128(int row, int col_elem) {
  const int unit = (col_elem >> 3) ^ (row & 7);
  return row * 128 + unit * 16 + (col_elem & 7) * 2;
}

// tok_seq[t], tok_pos[t]: sequence slot and position of packed token t. Copies the rotated K and
// the V rows of qkv[t] into the cache pages named by block_table[seq][pos / 128].
__global__ void kv_write_kernel(const __nv_bfloat16* __restrict__ qkv, __nv_bfloat16* __restrict__ kcache,
                                __nv_bfloat16* __restrict__ vcache, const int* __restrict__ tok_seq,
                                const int* __restrict__ tok_pos, const int* __restrict__ block_table,
                                int max_pages, long long T, int Hq, int Hkv, int num_pages) {
  const long long n = T * Hkv * 2;  // (token, k|v, head) items, 16 lanes x 16 B each
  const int sub = threadIdx.x & 15;
  for (long long item = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 4; item < n;
       item += ((long long)gridDim.x * blockDim.x) >> 4) {
    const long long t = item / (Hkv * 2);
    const int r = (int)(item - t * Hkv * 2);
    const int is_v = r / Hkv, hk = r - is_v * Hkv;
    const int seq = tok_seq[t], pos = tok_pos[t];
    if (seq < 0 || pos < 0) continue;
    AXB_DEBUG_CHECK(pos / PA_PAGE < max_pages, pos, max_pages);
    if (pos / PA_PAGE >= max_pages) continue;
    const int page = block_table[(long long)seq * max_pages + pos / PA_PAGE];
    AXB_DEBUG_CHECK(page >= 0 && page < num_pages, page, num_pages);
    if (page < 0 || page >= num_pages) continue;
    const __nv_bfloat16* src = qkv + t * (long long)(Hq + 2 * Hkv) * PA_D + (long long)(Hq + is_v * Hkv + hk) * PA_D;
    __nv_bfloat16* dst = (is_v ? vcache : kcache) +
                         (((long long)page * Hkv + hk) * PA_PAGE + (pos % PA_PAGE)) * PA_D;
    reinterpret_cast<uint4*>(dst)[sub] = reinterpret_cast<const uint4*>(src)[sub];
  }
}

__global__ void __launch_bounds__(128, 1)
paged_decode_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                    const __nv_bfloat16* __restrict__ q, long long q_row_stride,
                    const int* __restrict__ block_table, int max_pages, const int* __restrict__ seq_lens,
                    __nv_bfloat16* __restrict__ out, float* __restrict__ part_o, float* __restrict__ part_ml,
                    int Hq, int Hkv, int nsplit, float scale_log2, int* status) {
  grid_dependency_wait();
  grid_launch_dependents();   // the output projection (a programmatic dependent) may start streaming its weights
  const int hk = blockIdx.x, b = blockIdx.y, sp = blockIdx.z;
  const int rep = Hq / Hkv;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int seq_len = seq_lens[b];
  const int n_blocks = (seq_len + PA_PAGE - 1) / PA_PAGE;
  const int per = (n_blocks + nsplit - 1) / nsplit;
  const int blk_begin = sp * per;
  const int blk_end = min(n_blocks, blk_begin + per);
  const int nb = blk_end - blk_begin;
  if (nb <= 0) {
    if (nsplit > 1 && tid < rep) {
      const long long idx = ((long long)b * Hq + hk * rep + tid) * nsplit + sp;
      part_ml[idx * 2] = -1e30f;
      part_ml[idx * 2 + 1] = 0.f;
    }
    return;
  }

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sKV = smem;                                  // [stage][K 32K | V 32K]
  uint8_t* sQ = smem + PA_STAGES * 2 * PA_TILE;         // [2 chunks][16 rows][64] bf16
  uint8_t* sP = sQ + 4096;
  float* red = reinterpret_cast<float*>(sP + 4096);     // [2][4 warps][16]
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + 4096 + 1024);
  uint64_t* full = bars;                                // [PA_STAGES]
  uint64_t* bar_mma = bars + PA_STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + PA_STAGES + 1);

  if (tid == 0) {
    for (int s = 0; s < PA_STAGES; ++s) mbar_init(&full[s], 1);
    mbar_init(bar_mma, 1);
    mbar_fence_init();
  }
  if (warp == 0) {
    tmem_alloc(tmem_slot, 32);
    tmem_relinquish();
  }
  // Q^T operand: rows = heads of the group (zero padded to 16), K-major over the 128 dims.
  for (int i = tid; i < 4096 / 16; i += 128) reinterpret_cast<uint4*>(sQ)[i] = make_uint4(0, 0, 0, 0);
  __syncthreads();
  for (int hh = 0; hh < rep; ++hh) {
    const __nv_bfloat16 v = q[(long long)b * q_row_stride + (long long)(hk * rep + hh) * PA_D + tid];
    *reinterpret_cast<__nv_bfloat16*>(sQ + (tid >> 6) * 2048 + pa_sw128(hh, tid & 63)) = v;
  }
  fence_async_shared();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tS = tmem_base + (static_cast<uint32_t>(warp * 32) << 16);
  const uint32_t tO = tS + 16;
  constexpr uint32_t idesc_s = umma_idesc(128, PA_NPAD, 0, 0);
  constexpr uint32_t idesc_o = umma_idesc(128, PA_NPAD, 1, 0);
  const int* bt = block_table + (long long)b * max_pages;

  auto issue_load = [&](int i) {  // i-th block of this split -> stage i % STAGES
    const int s = i % PA_STAGES;
    const int page = bt[blk_begin + i];
    const int row0 = (page * Hkv + hk) * PA_PAGE;
    uint8_t* k = sKV + s * 2 * PA_TILE;
    mbar_expect_tx(&full[s], 2 * PA_TILE);
    tma_load_2d(k, &tmK, &full[s], 0, row0);
    tma_load_2d(k + 16384, &tmK, &full[s], 64, row0);
    tma_load_2d(k + PA_TILE, &tmV, &full[s], 0, row0);
    tma_load_2d(k + PA_TILE + 16384, &tmV, &full[s], 64, row0);
  };
  if (tid == 0) {
    for (int i = 0; i < PA_STAGES - 1 && i < nb; ++i) issue_load(i);
  }

  float m_run[8], l_thr[8];
#pragma unroll
  for (int hh = 0; hh < 8; ++hh) {
    m_run[hh] = -1e30f;
    l_thr[hh] = 0.f;
  }
  bool ok = true;
  uint32_t ph = 0;  // bar_mma completes once per block (after S) and once after the last P*V
  for (int i = 0; i < nb; ++i) {
    const int s = i % PA_STAGES;
    const uint32_t kaddr = smem_u32(sKV + s * 2 * PA_TILE);
    if (tid == 0 && ok) {
      if (!mbar_wait(&full[s], (i / PA_STAGES) & 1)) {
        report_error(status, AXB_ERR_WAIT_FULL);
        ok = false;
      }
      tc_fence_after();
      const uint32_t qaddr = smem_u32(sQ);
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        umma_f16_ss(tmem_base, umma_smem_desc(kaddr + (ks >> 2) * 16384 + (ks & 3) * 32, 16, 1024),
                    umma_smem_desc(qaddr + (ks >> 2) * 2048 + (ks & 3) * 32, 16, 1024), idesc_s, ks != 0);
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
    if (tid == 0 && ok && i + PA_STAGES - 1 < nb) issue_load(i + PA_STAGES - 1);

    uint32_t sv[16];
    tmem_ld_32x16(tS, sv);
    tmem_ld_wait();
    const int kpos = (blk_begin + i) * PA_PAGE + tid;
    const bool valid = kpos < seq_len;
    float sc[8];
#pragma unroll
    for (int hh = 0; hh < 8; ++hh) {
      sc[hh] = (valid && hh < rep) ? __uint_as_float(sv[hh]) * scale_log2 : -INFINITY;
      const float wm = warp_max(sc[hh]);
      if (lane == 0) red[((i & 1) * 4 + warp) * 16 + hh] = wm;
    }
    __syncthreads();
    float alpha[8];
    bool changed = false;
#pragma unroll
    for (int hh = 0; hh < 8; ++hh) {
      const float* r = red + (i & 1) * 64 + hh;
      const float bm = fmaxf(fmaxf(r[0], r[16]), fmaxf(r[32], r[48]));
      const float mn = fmaxf(m_run[hh], bm);
      alpha[hh] = exp2f(m_run[hh] - mn);
      changed |= (mn != m_run[hh]);
      m_run[hh] = mn;
      const float p = exp2f(sc[hh] - mn);
      l_thr[hh] = l_thr[hh] * alpha[hh] + p;
      if (hh < rep)
        *reinterpret_cast<__nv_bfloat16*>(sP + (tid >> 6) * 2048 + pa_sw128(hh, tid & 63)) = __float2bfloat16(p);
    }
    if (i > 0 && changed) {  // uniform across the CTA: m_run is identical in every thread
      uint32_t o[16];
      tmem_ld_32x16(tO, o);
      tmem_ld_wait();
#pragma unroll
      for (int hh = 0; hh < 8; ++hh) o[hh] = __float_as_uint(__uint_as_float(o[hh]) * alpha[hh]);
      asm volatile(
          "tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
          ::"r"(tO), "r"(o[0]), "r"(o[1]), "r"(o[2]), "r"(o[3]), "r"(o[4]), "r"(o[5]), "r"(o[6]), "r"(o[7])
          : "memory");
      tmem_st_wait();
    }
    fence_async_shared();
    tc_fence_before();
    __syncthreads();
    if (tid == 0 && ok) {
      tc_fence_after();
      const uint32_t vaddr = kaddr + PA_TILE, paddr = smem_u32(sP);
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        umma_f16_ss(tmem_base + 16, umma_smem_desc(vaddr + ks * 2048, 16384, 1024),
                    umma_smem_desc(paddr + (ks >> 2) * 2048 + (ks & 3) * 32, 16, 1024), idesc_o,
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

  // ---- epilogue. l per head: reduce the per-thread partial sums over the CTA.
  float l_tot[8];
#pragma unroll
  for (int hh = 0; hh < 8; ++hh) {
    const float ws = warp_sum(l_thr[hh]);
    if (lane == 0) red[warp * 16 + hh] = ws;
  }
  __syncthreads();
#pragma unroll
  for (int hh = 0; hh < 8; ++hh) l_tot[hh] = red[hh] + red[16 + hh] + red[32 + hh] + red[48 + hh];
  {
    uint32_t o[16];
    tmem_ld_32x16(tO, o);
    tmem_ld_wait();
    if (ok) {
#pragma unroll
      for (int hh = 0; hh < 8; ++hh) {
        if (hh < rep) {
          const int h = hk * rep + hh;
          const float v = __uint_as_float(o[hh]);
          if (nsplit == 1) {
            out[((long long)b * Hq + h) * PA_D + tid] = __float2bfloat16(v / l_tot[hh]);
          } else {
            const long long idx = ((long long)b * Hq + h) * nsplit + sp;
            part_o[idx * PA_D + tid] = v;
            if (tid == 0) {
              part_ml[idx * 2] = m_run[hh];
              part_ml[idx * 2 + 1] = l_tot[hh];
            }
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 32);
  }
}

// out[b][h][:] = sum_s O_s 2^(m_s - M) / sum_s l_s 2^(m_s - M)
__global__ void paged_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                   __nv_bfloat16* __restrict__ out, int nsplit) {
  grid_dependency_wait();
  grid_launch_dependents();
  const long long bh = blockIdx.x;
  const int d = threadIdx.x;
  float M = -1e30f;
  for (int s = 0; s < nsplit; ++s) M = fmaxf(M, part_ml[(bh * nsplit + s) * 2]);
  float acc = 0.f, l = 0.f;
  for (int s = 0; s < nsplit; ++s) {
    const float ls = part_ml[(bh * nsplit + s) * 2 + 1];
    if (ls == 0.f) continue;
    const float w = exp2f(part_ml[(bh * nsplit + s) * 2] - M);
    acc += part_o[(bh * nsplit + s) * PA_D + d] * w;
    l += ls * w;
  }
  out[bh * PA_D + d] = __float2bfloat16(l > 0.f ? acc / l : 0.f);
}

}  // namespace axb

using namespace axb;

extern "C" int axb_kv_write(const void* qkv, void* kcache, void* vcache, const int* tok_seq, const int* tok_pos,
                            const int* block_table, int max_pages, long long T, int Hq, int Hkv, int D,
                            int num_pages, void* stream) {
  if (D != PA_D || T <= 0) return AXB_LAUNCH_BAD_ARG;
  const long long threads = T * Hkv * 2 * 16;
  long long blocks = (threads + 255) / 256;
  const long long cap = (long long)sm_count() * 16;
  if (blocks > cap) blocks = cap;
  kv_write_kernel<<<(int)blocks, 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)qkv, (__nv_bfloat16*)kcache, (__nv_bfloat16*)vcache, tok_seq, tok_pos, block_table,
      max_pages, T, Hq, Hkv, num_pages);
  return check_launch();
}

// Number of key splits the decode kernel will use for a batch of B sequences.
extern "C" int axb_paged_decode_splits(int B, int Hkv, int max_blocks) {
  const int ctas = B * Hkv;
  const int target = 2 * sm_count();
  int ns = ctas >= target ? 1 : (target + ctas - 1) / ctas;
  if (ns > max_blocks) ns = max_blocks;
  if (ns > 32) ns = 32;
  return ns < 1 ? 1 : ns;
}

// q: bf16 [B][q_row_stride] with head h at column h*128. out: bf16 [B][Hq*128].
// kcache/vcache: [num_pages][Hkv][128][128]. scratch: when nsplit > 1,
// B*Hq*nsplit*(128+2)*4 bytes.
extern "C" int axb_paged_decode(const void* q, long long q_row_stride, const void* kcache, const void* vcache,
                                int num_pages, const int* block_table, int max_pages, const int* seq_lens,
                                void* out, int B, int Hq, int Hkv, int D, float softmax_scale, int nsplit,
                                void* scratch, int* status, void* stream) {
  if (D != PA_D || B <= 0 || Hq % Hkv != 0 || Hq / Hkv > 8 || nsplit < 1) return AXB_LAUNCH_BAD_ARG;
  cudaStream_t s = (cudaStream_t)stream;
  CUtensorMap tmK, tmV;
  const unsigned long long rows = (unsigned long long)num_pages * Hkv * PA_PAGE;
  int rc = make_tmap_2d(&tmK, kcache, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, PA_D, rows, PA_D * 2, 64, PA_PAGE, true);
  if (rc) return rc;
  rc = make_tmap_2d(&tmV, vcache, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, PA_D, rows, PA_D * 2, 64, PA_PAGE, true);
  if (rc) return rc;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(paged_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PA_SMEM) != cudaSuccess)
      return AXB_LAUNCH_CUDA_ERROR;
    attr_set = true;
  }
  float* part_o = reinterpret_cast<float*>(scratch);
  float* part_ml = part_o ? part_o + (long long)B * Hq * nsplit * PA_D : nullptr;
  if (nsplit > 1 && scratch == nullptr) return AXB_LAUNCH_BAD_ARG;
  rc = launch_dependent(paged_decode_kernel, dim3(Hkv, B, nsplit), dim3(128), PA_SMEM, s, tmK, tmV, (const __nv_bfloat16*)q,
                        q_row_stride, block_table, max_pages, seq_lens, (__nv_bfloat16*)out, part_o, part_ml, Hq, Hkv, nsplit,
                        softmax_scale * 1.4426950408889634f, status);
  if (!rc) rc = check_launch();
  if (rc || nsplit == 1) return rc;
  rc = launch_dependent(paged_merge_kernel, dim3(B * Hq), dim3(PA_D), 0, s, (const float*)part_o, (const float*)part_ml,
                        (__nv_bfloat16*)out, nsplit);
  return rc ? rc : check_launch();
}
