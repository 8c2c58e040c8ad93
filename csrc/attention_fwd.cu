// Packed (varlen) causal GQA attention forward on tcgen05 tensor cores, head dim 128.
//
// One CTA (128 threads) owns a 128-query tile of one sequence and one query head and walks
// the key blocks of that sequence:
//     S  = Q K^T        tcgen05.mma  -> TMEM columns [0,128)
//     P  = softmax tile thread t owns query row t (tcgen05.ld 32x32b), writes bf16 P into the
//                       K tile's shared memory in the swizzled K-major layout
//     O += P V          tcgen05.mma  -> TMEM columns [128,256)
// O stays in TMEM for the whole loop; it is rescaled only when the running row maximum grew by
// more than 2^8 since the last rescale (the row sum uses the same stale maximum, so the final
// O / l is exact). Two CTAs fit on an SM (96 KB shared memory, 256 TMEM columns each) and
// overlap each other's softmax and MMA phases. Q, K, V come through 3-D TMA maps over the
// packed [token][head][128] buffers, so GQA needs no repeat of K/V.
//
// Replaces flash-attn varlen in the reference's FSDP path (HF flash_attention_2,
// axon/trainer/fsdp_trainer.py:223-233).
#include "ptx.cuh"
#include "host_utils.h"

namespace axb {

constexpr int ATT_D = 128;
constexpr int ATT_BM = 128;
constexpr int ATT_BN = 128;
constexpr int ATT_TILE_BYTES = ATT_BM * ATT_D * 2;  // 32 KB
constexpr int ATT_SMEM = 3 * ATT_TILE_BYTES + 1024 + 128;

struct AttnTile {
  int seq_start;  // first packed token of the sequence
  int seq_len;
  int q_blk;      // 128-row block inside the sequence
  int pad;
};

// tiles[0..count) for all sequences, heaviest (last) query blocks first inside a sequence.
__global__ void build_attn_tiles_kernel(const int* __restrict__ cu_seqlens, int B, AttnTile* tiles,
                                        int* count, int max_tiles) {
  if (blockIdx.x != 0 || threadIdx.x != 0) return;
  int n = 0;
  for (int b = 0; b < B; ++b) {
    const int s = cu_seqlens[b], len = cu_seqlens[b + 1] - s;
    const int nb = (len + ATT_BM - 1) / ATT_BM;
    for (int qb = nb - 1; qb >= 0 && n < max_tiles; --qb) tiles[n++] = AttnTile{s, len, qb, 0};
  }
  *count = n;
}

__device__ __forceinline__ uint32_t sw128_offset(int row, int col_elem) {
  // byte offset of bf16 element (row, col) inside a [rows][64]-element 128B-swizzled chunk
  const int unit = (col_elem >> 3) ^ (row & 7);
  return row * 128 + unit * 16 + (col_elem & 7) * 2;
}

__global__ void __launch_bounds__(128, 2)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, __nv_bfloat16* __restrict__ O,
                float* __restrict__ LSE, const AttnTile* __restrict__ tiles,
                const int* __restrict__ tile_count, int Hq, int Hkv, long long o_row_stride, int T,
                float scale_log2, int causal, int* status) {
  const int tile_id = blockIdx.y;
  if (tile_id >= *tile_count) return;
  const AttnTile tile = tiles[tile_id];
  const int h = blockIdx.x;
  const int hk = h / (Hq / Hkv);
  const int q0 = tile.q_blk * ATT_BM;  // position of row 0 inside the sequence

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sQ = smem;
  uint8_t* sK = smem + ATT_TILE_BYTES;  // also holds P after S is computed
  uint8_t* sV = smem + 2 * ATT_TILE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 3 * ATT_TILE_BYTES);
  uint64_t* bar_q = bars;
  uint64_t* bar_k = bars + 1;
  uint64_t* bar_v = bars + 2;
  uint64_t* bar_mma = bars + 3;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 4);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) {
    mbar_init(bar_q, 1);
    mbar_init(bar_k, 1);
    mbar_init(bar_v, 1);
    mbar_init(bar_mma, 1);
    mbar_fence_init();
  }
  if (warp == 0) {
    tmem_alloc(tmem_slot, 256);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tS = tmem_base + (static_cast<uint32_t>(warp * 32) << 16);
  const uint32_t tO = tS + 128;

  const int kv_end = causal ? min(tile.seq_len, q0 + ATT_BM) : tile.seq_len;
  const int n_kv = (kv_end + ATT_BN - 1) / ATT_BN;
  constexpr uint32_t idesc_s = umma_idesc(128, 128, 0, 0);
  constexpr uint32_t idesc_o = umma_idesc(128, 128, 0, 1);

  if (tid == 0) {
    mbar_expect_tx(bar_q, ATT_TILE_BYTES);
    tma_load_3d(sQ, &tmQ, bar_q, 0, h, tile.seq_start + q0);
    tma_load_3d(sQ + 16384, &tmQ, bar_q, 64, h, tile.seq_start + q0);
  }

  const int row = tid;            // query row inside the tile
  const int qpos = q0 + row;      // position inside the sequence
  float m_used = -1e30f, l_sum = 0.f;
  bool ok = true;

  for (int j = 0; j < n_kv; ++j) {
    const int k0 = j * ATT_BN;
    if (tid == 0 && ok) {
      mbar_expect_tx(bar_k, ATT_TILE_BYTES);
      tma_load_3d(sK, &tmK, bar_k, 0, hk, tile.seq_start + k0);
      tma_load_3d(sK + 16384, &tmK, bar_k, 64, hk, tile.seq_start + k0);
      mbar_expect_tx(bar_v, ATT_TILE_BYTES);
      tma_load_3d(sV, &tmV, bar_v, 0, hk, tile.seq_start + k0);
      tma_load_3d(sV + 16384, &tmV, bar_v, 64, hk, tile.seq_start + k0);
      bool w = (j > 0) || mbar_wait(bar_q, 0);
      w = w && mbar_wait(bar_k, j & 1);
      if (!w) {
        report_error(status, AXB_ERR_WAIT_FULL);
        ok = false;
      }
      tc_fence_after();
      const uint32_t a0 = smem_u32(sQ), b0 = smem_u32(sK);
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        const uint32_t off = (ks >> 2) * 16384 + (ks & 3) * 32;
        umma_f16_ss(tmem_base, umma_smem_desc(a0 + off, 16, 1024), umma_smem_desc(b0 + off, 16, 1024),
                    idesc_s, ks != 0);
      }
      tc_commit(bar_mma);
    }
    __syncwarp();
    if (ok && !mbar_wait(bar_mma, 0)) {
      report_error(status, AXB_ERR_WAIT_TMEM_FULL);
      ok = false;
    }
    tc_fence_after();

    // ---- softmax on this thread's row
    uint32_t s[4][32];
#pragma unroll
    for (int c = 0; c < 4; ++c) tmem_ld_32x32(tS + c * 32, s[c]);
    tmem_ld_wait();
    const bool need_mask = (k0 + ATT_BN > tile.seq_len) || (causal && k0 + ATT_BN - 1 > q0);
    float mx = -INFINITY;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        float v = __uint_as_float(s[c][i]) * scale_log2;
        if (need_mask) {
          const int kpos = k0 + c * 32 + i;
          if (kpos >= tile.seq_len || (causal && kpos > qpos)) v = -INFINITY;
        }
        s[c][i] = __float_as_uint(v);
        mx = fmaxf(mx, v);
      }
    }
    float alpha = 1.f;
    bool rescale = false;
    if (j == 0) {
      m_used = fmaxf(mx, -1e30f);
    } else if (mx > m_used + 8.f) {
      alpha = exp2f(m_used - mx);
      m_used = mx;
      rescale = true;
    }
    if (__any_sync(0xffffffffu, rescale)) {
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t o[32];
        tmem_ld_32x32(tO + c * 32, o);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
        tmem_st_32x32(tO + c * 32, o);
      }
      tmem_st_wait();
      l_sum *= alpha;
    }
    float rs = 0.f;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        float p[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          p[i] = exp2f(__uint_as_float(s[c][u * 8 + i]) - m_used);
          rs += p[i];
        }
        uint4 v;
        v.x = pack_bf16x2(p[0], p[1]);
        v.y = pack_bf16x2(p[2], p[3]);
        v.z = pack_bf16x2(p[4], p[5]);
        v.w = pack_bf16x2(p[6], p[7]);
        const int col = c * 32 + u * 8;  // key column inside the block
        uint8_t* dst = sK + (col >> 6) * 16384 + sw128_offset(row, col & 63);
        *reinterpret_cast<uint4*>(dst) = v;
      }
    }
    l_sum += rs;
    fence_async_shared();
    tc_fence_before();
    __syncthreads();

    if (tid == 0 && ok) {
      if (!mbar_wait(bar_v, j & 1)) report_error(status, AXB_ERR_WAIT_FULL);
      tc_fence_after();
      const uint32_t a0 = smem_u32(sK), b0 = smem_u32(sV);
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        const uint32_t aoff = (ks >> 2) * 16384 + (ks & 3) * 32;
        umma_f16_ss(tmem_base + 128, umma_smem_desc(a0 + aoff, 16, 1024),
                    umma_smem_desc(b0 + ks * 2048, 16384, 1024), idesc_o, (j | ks) != 0);
      }
      tc_commit(bar_mma);
    }
    __syncwarp();
    if (ok && !mbar_wait(bar_mma, 1)) {
      report_error(status, AXB_ERR_WAIT_TMEM_FULL);
      ok = false;
    }
    tc_fence_after();
  }

  // ---- epilogue: O / l -> bf16, LSE
  if (ok && n_kv > 0) {
    const float inv_l = 1.f / l_sum;
    const bool valid = qpos < tile.seq_len;
    const long long tok = (long long)tile.seq_start + qpos;
    __nv_bfloat16* orow = O + tok * o_row_stride + (long long)h * ATT_D;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      uint32_t o[32];
      tmem_ld_32x32(tO + c * 32, o);
      tmem_ld_wait();
      if (valid) {
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          uint4 v;
          v.x = pack_bf16x2(__uint_as_float(o[u * 8 + 0]) * inv_l, __uint_as_float(o[u * 8 + 1]) * inv_l);
          v.y = pack_bf16x2(__uint_as_float(o[u * 8 + 2]) * inv_l, __uint_as_float(o[u * 8 + 3]) * inv_l);
          v.z = pack_bf16x2(__uint_as_float(o[u * 8 + 4]) * inv_l, __uint_as_float(o[u * 8 + 5]) * inv_l);
          v.w = pack_bf16x2(__uint_as_float(o[u * 8 + 6]) * inv_l, __uint_as_float(o[u * 8 + 7]) * inv_l);
          reinterpret_cast<uint4*>(orow + c * 32)[u] = v;
        }
      }
    }
    if (valid && LSE != nullptr)
      LSE[(long long)h * T + tok] = (m_used + log2f(l_sum)) * 0.6931471805599453f;
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 256);
  }
}

}  // namespace axb

using namespace axb;

extern "C" int axb_attn_max_tiles(long long T, int B) { return (int)(T / ATT_BM + B + 1); }

// q/k/v: bf16 packed [T][row_stride] with head h at column h*128 (they may alias one fused
// qkv buffer). o: bf16 [T][o_row_stride]. lse: fp32 [Hq][T] or null. cu_seqlens: int32 [B+1] on
// the device. tiles_scratch: axb_attn_max_tiles(T,B) * 16 bytes + 16 bytes (device).
extern "C" int axb_attn_fwd(const void* q, const void* k, const void* v, void* o, float* lse,
                            const int* cu_seqlens, int B, long long T, int Hq, int Hkv, int D,
                            long long q_row_stride, long long kv_row_stride, long long o_row_stride,
                            float softmax_scale, int causal, void* tiles_scratch, int* status,
                            void* stream) {
  if (D != ATT_D || T <= 0 || B <= 0 || Hq % Hkv != 0) return AXB_LAUNCH_BAD_ARG;
  if ((o_row_stride & 7) != 0) return AXB_LAUNCH_BAD_ARG;
  cudaStream_t s = (cudaStream_t)stream;
  const int max_tiles = axb_attn_max_tiles(T, B);
  int* count = reinterpret_cast<int*>(tiles_scratch);
  AttnTile* tiles = reinterpret_cast<AttnTile*>(reinterpret_cast<uint8_t*>(tiles_scratch) + 16);
  build_attn_tiles_kernel<<<1, 1, 0, s>>>(cu_seqlens, B, tiles, count, max_tiles);
  int rc = check_launch();
  if (rc) return rc;
  CUtensorMap tmQ, tmK, tmV;
  rc = make_tmap_3d(&tmQ, q, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, ATT_D, Hq, T, ATT_D * 2,
                    q_row_stride * 2, 64, 1, ATT_BM, true);
  if (rc) return rc;
  rc = make_tmap_3d(&tmK, k, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, ATT_D, Hkv, T, ATT_D * 2,
                    kv_row_stride * 2, 64, 1, ATT_BN, true);
  if (rc) return rc;
  rc = make_tmap_3d(&tmV, v, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, ATT_D, Hkv, T, ATT_D * 2,
                    kv_row_stride * 2, 64, 1, ATT_BN, true);
  if (rc) return rc;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(attn_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, ATT_SMEM) !=
        cudaSuccess)
      return AXB_LAUNCH_CUDA_ERROR;
    attr_set = true;
  }
  dim3 grid(Hq, max_tiles);
  attn_fwd_kernel<<<grid, 128, ATT_SMEM, s>>>(tmQ, tmK, tmV, (__nv_bfloat16*)o, lse, tiles, count, Hq,
                                             Hkv, o_row_stride, (int)T,
                                             softmax_scale * 1.4426950408889634f, causal, status);
  return check_launch();
}
