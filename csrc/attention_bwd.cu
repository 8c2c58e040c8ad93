// Packed causal GQA attention backward on tcgen05, head dim 128. Deterministic (no atomics):
//
//   attn_delta_kernel   delta[h][t] = sum_d O[t,h,d] * dO[t,h,d]
//   attn_bwd_dkv_kernel one CTA per (key block, kv head): loops over the query heads of the
//                       group and the query blocks at or below the diagonal;
//                       dV += P^T dO and dK += dS^T Q accumulate in TMEM across the whole loop.
//   attn_bwd_dq_kernel  one CTA per (query block, query head): loops over key blocks,
//                       dQ += dS K accumulates in TMEM (S and dP are recomputed).
//
// In both kernels thread t owns query row t of the S/dP tiles (tcgen05.ld 32x32b), computes
//   P = exp2(S*scale*log2e - LSE*log2e),  dS = P * (dP - delta) * scale
// and writes P / dS as bf16 into 128-byte-swizzled shared memory, which the next MMAs read
// either K-major (dS K) or MN-major (P^T dO, dS^T Q) without a transpose.
#include "ptx.cuh"
#include "host_utils.h"

namespace axb {

constexpr int AB_D = 128;
constexpr int AB_BLK = 128;
constexpr int AB_TILE = AB_BLK * AB_D * 2;  // 32 KB

struct AttnTile {
  int seq_start;
  int seq_len;
  int q_blk;
  int pad;
};

__device__ __forceinline__ uint32_t sw128_off(int row, int col_elem) {
  const int unit = (col_elem >> 3) ^ (row & 7);
  return row * 128 + unit * 16 + (col_elem & 7) * 2;
}

__global__ void attn_delta_kernel(const __nv_bfloat16* __restrict__ O, const __nv_bfloat16* __restrict__ dO,
                                  float* __restrict__ delta, long long T, int Hq, long long row_stride) {
  const int lane = threadIdx.x & 31;
  const long long n = T * Hq;
  for (long long item = (long long)blockIdx.x * 8 + (threadIdx.x >> 5); item < n;
       item += (long long)gridDim.x * 8) {
    const long long t = item / Hq;
    const int h = (int)(item - t * Hq);
    const uint2 a = *reinterpret_cast<const uint2*>(O + t * row_stride + h * AB_D + lane * 4);
    const uint2 b = *reinterpret_cast<const uint2*>(dO + t * row_stride + h * AB_D + lane * 4);
    const float2 a0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&a.x));
    const float2 a1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&a.y));
    const float2 b0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&b.x));
    const float2 b1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&b.y));
    float s = a0.x * b0.x + a0.y * b0.y + a1.x * b1.x + a1.y * b1.y;
    s = warp_sum(s);
    if (lane == 0) delta[(long long)h * T + t] = s;
  }
}

// Reads this thread's row of S and dP from TMEM, writes P and dS (bf16, swizzled [row][key]).
// k0: first key position of the block inside the sequence; qpos: this row's position.
__device__ __forceinline__ void softmax_grad_row(uint32_t tS, uint32_t tDP, uint8_t* sP, uint8_t* sDS,
                                                 int row, int qpos, int k0, int seq_len, int causal,
                                                 float lse2, float delta, float scale, float scale_log2) {
  const bool row_valid = qpos < seq_len;
#pragma unroll 1
  for (int c = 0; c < 4; ++c) {
    uint32_t s[32], dp[32];
    tmem_ld_32x32(tS + c * 32, s);
    tmem_ld_32x32(tDP + c * 32, dp);
    tmem_ld_wait();
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      float p[8], ds[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int kpos = k0 + c * 32 + u * 8 + i;
        const bool valid = row_valid && kpos < seq_len && (!causal || kpos <= qpos);
        const float pv = valid ? exp2f(__uint_as_float(s[u * 8 + i]) * scale_log2 - lse2) : 0.f;
        p[i] = pv;
        ds[i] = pv * (__uint_as_float(dp[u * 8 + i]) - delta) * scale;
      }
      uint4 vp, vd;
      vp.x = pack_bf16x2(p[0], p[1]); vp.y = pack_bf16x2(p[2], p[3]);
      vp.z = pack_bf16x2(p[4], p[5]); vp.w = pack_bf16x2(p[6], p[7]);
      vd.x = pack_bf16x2(ds[0], ds[1]); vd.y = pack_bf16x2(ds[2], ds[3]);
      vd.z = pack_bf16x2(ds[4], ds[5]); vd.w = pack_bf16x2(ds[6], ds[7]);
      const int col = c * 32 + u * 8;
      const uint32_t off = (col >> 6) * 16384 + sw128_off(row, col & 63);
      if (sP != nullptr) *reinterpret_cast<uint4*>(sP + off) = vp;
      *reinterpret_cast<uint4*>(sDS + off) = vd;
    }
  }
}

// Issue the 8 K-steps of a 128x128x128 product. a_mn/b_mn choose operand addressing:
//   K-major : 2 chunks of 64 along K, 32 B per K-step inside a chunk
//   MN-major: chunks of 64 along M/N (lbo 16384), 2048 B per K-step
__device__ __forceinline__ void mma_128x128x128(uint32_t d_tmem, uint32_t a_base, bool a_mn, uint32_t b_base,
                                                bool b_mn, uint32_t idesc, bool accumulate_first) {
#pragma unroll
  for (int ks = 0; ks < 8; ++ks) {
    const uint32_t koff = (ks >> 2) * 16384 + (ks & 3) * 32;
    const uint64_t ad = a_mn ? umma_smem_desc(a_base + ks * 2048, 16384, 1024)
                             : umma_smem_desc(a_base + koff, 16, 1024);
    const uint64_t bd = b_mn ? umma_smem_desc(b_base + ks * 2048, 16384, 1024)
                             : umma_smem_desc(b_base + koff, 16, 1024);
    umma_f16_ss(d_tmem, ad, bd, idesc, (accumulate_first || ks != 0) ? 1u : 0u);
  }
}

__device__ __forceinline__ void load_tile(uint8_t* dst, const CUtensorMap* tm, uint64_t* bar, int head, int tok) {
  tma_load_3d(dst, tm, bar, 0, head, tok);
  tma_load_3d(dst + 16384, tm, bar, 64, head, tok);
}

constexpr int AB_DKV_SMEM = 6 * AB_TILE + 1024 + 128;
constexpr int AB_DQ_SMEM = 5 * AB_TILE + 1024 + 128;

__global__ void __launch_bounds__(128, 1)
attn_bwd_dkv_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                    const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO,
                    const float* __restrict__ LSE, const float* __restrict__ DELTA,
                    __nv_bfloat16* __restrict__ dK, __nv_bfloat16* __restrict__ dV,
                    const AttnTile* __restrict__ tiles, const int* __restrict__ tile_count, int Hq, int Hkv,
                    long long dkv_row_stride, int T, float scale, int causal, int* status) {
  const int tile_id = blockIdx.y;
  if (tile_id >= *tile_count) return;
  const AttnTile tile = tiles[tile_id];
  const int hk = blockIdx.x;
  const int rep = Hq / Hkv;
  const int k0 = tile.q_blk * AB_BLK;
  const int n_qblk = (tile.seq_len + AB_BLK - 1) / AB_BLK;
  const int i_begin = causal ? tile.q_blk : 0;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sK = smem;
  uint8_t* sV = smem + AB_TILE;
  uint8_t* sQ = smem + 2 * AB_TILE;
  uint8_t* sDO = smem + 3 * AB_TILE;
  uint8_t* sP = smem + 4 * AB_TILE;
  uint8_t* sDS = smem + 5 * AB_TILE;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 6 * AB_TILE);
  uint64_t* bar_kv = bars;
  uint64_t* bar_q = bars + 1;
  uint64_t* bar_mma = bars + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 3);

  const int tid = threadIdx.x, warp = tid >> 5;
  if (tid == 0) {
    mbar_init(bar_kv, 1);
    mbar_init(bar_q, 1);
    mbar_init(bar_mma, 1);
    mbar_fence_init();
  }
  if (warp == 0) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t lane_off = static_cast<uint32_t>(warp * 32) << 16;
  const uint32_t tS = tmem_base + lane_off, tDP = tS + 128, tDV = tS + 256, tDK = tS + 384;
  constexpr uint32_t idesc_kk = umma_idesc(128, 128, 0, 0);
  constexpr uint32_t idesc_mm = umma_idesc(128, 128, 1, 1);
  const float scale_log2 = scale * 1.4426950408889634f;

  if (tid == 0) {
    mbar_expect_tx(bar_kv, 2 * AB_TILE);
    load_tile(sK, &tmK, bar_kv, hk, tile.seq_start + k0);
    load_tile(sV, &tmV, bar_kv, hk, tile.seq_start + k0);
  }
  bool ok = true;
  int it = 0;
  for (int hr = 0; hr < rep; ++hr) {
    const int h = hk * rep + hr;
    for (int i = i_begin; i < n_qblk; ++i, ++it) {
      const int q0 = i * AB_BLK;
      if (tid == 0 && ok) {
        mbar_expect_tx(bar_q, 2 * AB_TILE);
        load_tile(sQ, &tmQ, bar_q, h, tile.seq_start + q0);
        load_tile(sDO, &tmDO, bar_q, h, tile.seq_start + q0);
        bool w = (it > 0) || mbar_wait(bar_kv, 0);
        w = w && mbar_wait(bar_q, it & 1);
        if (!w) {
          report_error(status, AXB_ERR_WAIT_FULL);
          ok = false;
        }
        tc_fence_after();
        mma_128x128x128(tmem_base, smem_u32(sQ), false, smem_u32(sK), false, idesc_kk, false);
        mma_128x128x128(tmem_base + 128, smem_u32(sDO), false, smem_u32(sV), false, idesc_kk, false);
        tc_commit(bar_mma);
      }
      __syncwarp();
      if (ok && !mbar_wait(bar_mma, 0)) {
        report_error(status, AXB_ERR_WAIT_TMEM_FULL);
        ok = false;
      }
      tc_fence_after();
      const int qpos = q0 + tid;
      const long long tok = (long long)tile.seq_start + qpos;
      const bool in_range = qpos < tile.seq_len && tok < T;
      const float lse2 = in_range ? LSE[(long long)h * T + tok] * 1.4426950408889634f : 0.f;
      const float dl = in_range ? DELTA[(long long)h * T + tok] : 0.f;
      softmax_grad_row(tS, tDP, sP, sDS, tid, qpos, k0, tile.seq_len, causal, lse2, dl, scale, scale_log2);
      fence_async_shared();
      tc_fence_before();
      __syncthreads();
      if (tid == 0 && ok) {
        tc_fence_after();
        mma_128x128x128(tmem_base + 256, smem_u32(sP), true, smem_u32(sDO), true, idesc_mm, it > 0);
        mma_128x128x128(tmem_base + 384, smem_u32(sDS), true, smem_u32(sQ), true, idesc_mm, it > 0);
        tc_commit(bar_mma);
      }
      __syncwarp();
      if (ok && !mbar_wait(bar_mma, 1)) {
        report_error(status, AXB_ERR_WAIT_TMEM_FULL);
        ok = false;
      }
      tc_fence_after();
    }
  }
  // epilogue: thread = key row
  {
    const int kpos = k0 + tid;
    const bool valid = ok && it > 0 && kpos < tile.seq_len;
    const long long tok = (long long)tile.seq_start + kpos;
#pragma unroll 1
    for (int which = 0; which < 2; ++which) {
      const uint32_t src = which == 0 ? tDV : tDK;
      __nv_bfloat16* dst = (which == 0 ? dV : dK) + tok * dkv_row_stride + (long long)hk * AB_D;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t o[32];
        tmem_ld_32x32(src + c * 32, o);
        tmem_ld_wait();
        if (valid) {
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            uint4 v;
            v.x = pack_bf16x2(__uint_as_float(o[u * 8 + 0]), __uint_as_float(o[u * 8 + 1]));
            v.y = pack_bf16x2(__uint_as_float(o[u * 8 + 2]), __uint_as_float(o[u * 8 + 3]));
            v.z = pack_bf16x2(__uint_as_float(o[u * 8 + 4]), __uint_as_float(o[u * 8 + 5]));
            v.w = pack_bf16x2(__uint_as_float(o[u * 8 + 6]), __uint_as_float(o[u * 8 + 7]));
            reinterpret_cast<uint4*>(dst + c * 32)[u] = v;
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

__global__ void __launch_bounds__(128, 1)
attn_bwd_dq_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                   const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO,
                   const float* __restrict__ LSE, const float* __restrict__ DELTA,
                   __nv_bfloat16* __restrict__ dQ, const AttnTile* __restrict__ tiles,
                   const int* __restrict__ tile_count, int Hq, int Hkv, long long dq_row_stride, int T,
                   float scale, int causal, int* status) {
  const int tile_id = blockIdx.y;
  if (tile_id >= *tile_count) return;
  const AttnTile tile = tiles[tile_id];
  const int h = blockIdx.x;
  const int hk = h / (Hq / Hkv);
  const int q0 = tile.q_blk * AB_BLK;
  const int kv_end = causal ? min(tile.seq_len, q0 + AB_BLK) : tile.seq_len;
  const int n_kv = (kv_end + AB_BLK - 1) / AB_BLK;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sQ = smem;
  uint8_t* sDO = smem + AB_TILE;
  uint8_t* sK = smem + 2 * AB_TILE;
  uint8_t* sV = smem + 3 * AB_TILE;
  uint8_t* sDS = smem + 4 * AB_TILE;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 5 * AB_TILE);
  uint64_t* bar_q = bars;
  uint64_t* bar_kv = bars + 1;
  uint64_t* bar_mma = bars + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 3);

  const int tid = threadIdx.x, warp = tid >> 5;
  if (tid == 0) {
    mbar_init(bar_q, 1);
    mbar_init(bar_kv, 1);
    mbar_init(bar_mma, 1);
    mbar_fence_init();
  }
  if (warp == 0) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t lane_off = static_cast<uint32_t>(warp * 32) << 16;
  const uint32_t tS = tmem_base + lane_off, tDP = tS + 128, tDQ = tS + 256;
  constexpr uint32_t idesc_kk = umma_idesc(128, 128, 0, 0);
  constexpr uint32_t idesc_km = umma_idesc(128, 128, 0, 1);
  const float scale_log2 = scale * 1.4426950408889634f;

  if (tid == 0) {
    mbar_expect_tx(bar_q, 2 * AB_TILE);
    load_tile(sQ, &tmQ, bar_q, h, tile.seq_start + q0);
    load_tile(sDO, &tmDO, bar_q, h, tile.seq_start + q0);
  }
  const int qpos = q0 + tid;
  const long long tok = (long long)tile.seq_start + qpos;
  const bool in_range = qpos < tile.seq_len && tok < T;
  const float lse2 = in_range ? LSE[(long long)h * T + tok] * 1.4426950408889634f : 0.f;
  const float dl = in_range ? DELTA[(long long)h * T + tok] : 0.f;
  bool ok = true;
  for (int j = 0; j < n_kv; ++j) {
    const int k0 = j * AB_BLK;
    if (tid == 0 && ok) {
      mbar_expect_tx(bar_kv, 2 * AB_TILE);
      load_tile(sK, &tmK, bar_kv, hk, tile.seq_start + k0);
      load_tile(sV, &tmV, bar_kv, hk, tile.seq_start + k0);
      bool w = (j > 0) || mbar_wait(bar_q, 0);
      w = w && mbar_wait(bar_kv, j & 1);
      if (!w) {
        report_error(status, AXB_ERR_WAIT_FULL);
        ok = false;
      }
      tc_fence_after();
      mma_128x128x128(tmem_base, smem_u32(sQ), false, smem_u32(sK), false, idesc_kk, false);
      mma_128x128x128(tmem_base + 128, smem_u32(sDO), false, smem_u32(sV), false, idesc_kk, false);
      tc_commit(bar_mma);
    }
    __syncwarp();
    if (ok && !mbar_wait(bar_mma, 0)) {
      report_error(status, AXB_ERR_WAIT_TMEM_FULL);
      ok = false;
    }
    tc_fence_after();
    softmax_grad_row(tS, tDP, nullptr, sDS, tid, qpos, k0, tile.seq_len, causal, lse2, dl, scale, scale_log2);
    fence_async_shared();
    tc_fence_before();
    __syncthreads();
    if (tid == 0 && ok) {
      tc_fence_after();
      mma_128x128x128(tmem_base + 256, smem_u32(sDS), false, smem_u32(sK), true, idesc_km, j > 0);
      tc_commit(bar_mma);
    }
    __syncwarp();
    if (ok && !mbar_wait(bar_mma, 1)) {
      report_error(status, AXB_ERR_WAIT_TMEM_FULL);
      ok = false;
    }
    tc_fence_after();
  }
  {
    const bool valid = ok && n_kv > 0 && qpos < tile.seq_len;
    __nv_bfloat16* dst = dQ + tok * dq_row_stride + (long long)h * AB_D;
#pragma unroll 1
    for (int c = 0; c < 4; ++c) {
      uint32_t o[32];
      tmem_ld_32x32(tDQ + c * 32, o);
      tmem_ld_wait();
      if (valid) {
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          uint4 v;
          v.x = pack_bf16x2(__uint_as_float(o[u * 8 + 0]), __uint_as_float(o[u * 8 + 1]));
          v.y = pack_bf16x2(__uint_as_float(o[u * 8 + 2]), __uint_as_float(o[u * 8 + 3]));
          v.z = pack_bf16x2(__uint_as_float(o[u * 8 + 4]), __uint_as_float(o[u * 8 + 5]));
          v.w = pack_bf16x2(__uint_as_float(o[u * 8 + 6]), __uint_as_float(o[u * 8 + 7]));
          reinterpret_cast<uint4*>(dst + c * 32)[u] = v;
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

__global__ void build_tiles_kernel(const int* __restrict__ cu_seqlens, int B, AttnTile* tiles, int* count,
                                   int max_tiles) {
  if (blockIdx.x != 0 || threadIdx.x != 0) return;
  int n = 0;
  for (int b = 0; b < B; ++b) {
    const int s = cu_seqlens[b], len = cu_seqlens[b + 1] - s;
    const int nb = (len + AB_BLK - 1) / AB_BLK;
    for (int qb = nb - 1; qb >= 0 && n < max_tiles; --qb) tiles[n++] = AttnTile{s, len, qb, 0};
  }
  *count = n;
}

}  // namespace axb

using namespace axb;

// q/k/v, dq/dk/dv: head slices of fused [T][row_stride] buffers (bf16); o/do: [T][o_row_stride].
// lse: fp32 [Hq][T] from the forward pass; delta: fp32 [Hq][T] scratch written here.
extern "C" int axb_attn_bwd(const void* q, const void* k, const void* v, const void* o, const void* d_o,
                            const float* lse, float* delta, void* dq, void* dk, void* dv,
                            const int* cu_seqlens, int B, long long T, int Hq, int Hkv, int D,
                            long long row_stride, long long o_row_stride, float softmax_scale, int causal,
                            void* tiles_scratch, int* status, void* stream) {
  if (D != AB_D || T <= 0 || B <= 0 || Hq % Hkv != 0) return AXB_LAUNCH_BAD_ARG;
  if ((row_stride & 7) != 0 || (o_row_stride & 7) != 0) return AXB_LAUNCH_BAD_ARG;
  cudaStream_t s = (cudaStream_t)stream;
  const int max_tiles = (int)(T / AB_BLK + B + 1);
  int* count = reinterpret_cast<int*>(tiles_scratch);
  AttnTile* tiles = reinterpret_cast<AttnTile*>(reinterpret_cast<uint8_t*>(tiles_scratch) + 16);
  build_tiles_kernel<<<1, 1, 0, s>>>(cu_seqlens, B, tiles, count, max_tiles);
  int rc = check_launch();
  if (rc) return rc;
  {
    long long items = T * Hq;
    long long blocks = (items + 7) / 8;
    long long cap = (long long)sm_count() * 16;
    attn_delta_kernel<<<(int)(blocks > cap ? cap : blocks), 256, 0, s>>>(
        (const __nv_bfloat16*)o, (const __nv_bfloat16*)d_o, delta, T, Hq, o_row_stride);
    rc = check_launch();
    if (rc) return rc;
  }
  CUtensorMap tmQ, tmK, tmV, tmDO;
  const CUtensorMapDataType bf = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  if ((rc = make_tmap_3d(&tmQ, q, bf, AB_D, Hq, T, AB_D * 2, row_stride * 2, 64, 1, AB_BLK, true))) return rc;
  if ((rc = make_tmap_3d(&tmK, k, bf, AB_D, Hkv, T, AB_D * 2, row_stride * 2, 64, 1, AB_BLK, true))) return rc;
  if ((rc = make_tmap_3d(&tmV, v, bf, AB_D, Hkv, T, AB_D * 2, row_stride * 2, 64, 1, AB_BLK, true))) return rc;
  if ((rc = make_tmap_3d(&tmDO, d_o, bf, AB_D, Hq, T, AB_D * 2, o_row_stride * 2, 64, 1, AB_BLK, true))) return rc;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(attn_bwd_dkv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, AB_DKV_SMEM) != cudaSuccess ||
        cudaFuncSetAttribute(attn_bwd_dq_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, AB_DQ_SMEM) != cudaSuccess)
      return AXB_LAUNCH_CUDA_ERROR;
    attr_set = true;
  }
  attn_bwd_dkv_kernel<<<dim3(Hkv, max_tiles), 128, AB_DKV_SMEM, s>>>(
      tmQ, tmK, tmV, tmDO, lse, delta, (__nv_bfloat16*)dk, (__nv_bfloat16*)dv, tiles, count, Hq, Hkv,
      row_stride, (int)T, softmax_scale, causal, status);
  rc = check_launch();
  if (rc) return rc;
  attn_bwd_dq_kernel<<<dim3(Hq, max_tiles), 128, AB_DQ_SMEM, s>>>(
      tmQ, tmK, tmV, tmDO, lse, delta, (__nv_bfloat16*)dq, tiles, count, Hq, Hkv, row_stride, (int)T,
      softmax_scale, causal, status);
  return check_launch();
}
