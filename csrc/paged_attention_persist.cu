// Persistent form of the item-based paged decode attention (paged_attention_shared.cu).
//
// The item kernels launch one CTA per (item, kv head, key split). With short items - the private tail of a
// sample after its shared prompt is a handful of pages - every CTA spends as long on start-up (TMEM allocation,
// barrier initialisation, the query load's global-memory latency, filling an empty TMA pipeline) as on its keys,
// which is why attention over shared prompt pages read 2.4x fewer bytes but ran only 7 % faster.
//
// Here ONE CTA per SM lives for the whole launch and pulls work units (item, kv head, split) from an atomic
// counter. TMEM is allocated once and the barriers are initialised once; the K|V tile ring keeps running
// ACROSS units (while the last tiles of a unit are being consumed, the first tiles of the next unit are already
// in flight), and the next unit's query rows are fetched with cp.async while the current unit computes. The tile
// mathematics is that of the item kernel: S^T = K_tile Q^T and O^T += V_tile^T P^T on tcgen05 with N = query
// columns, thread t owns key t for the softmax and output dimension t in the epilogue, lazily raised running
// maximum, un-normalised partial results per (sequence, head, slot) merged by paged_merge_slots_kernel.
//
// Every wait is bounded; a wait that runs out records a status code, drains the loads still in flight (bounded),
// frees TMEM and returns.
#include "ptx.cuh"
#include "host_utils.h"

namespace axb {

constexpr int PP_D = 128;
constexpr int PP_PAGE = 128;
constexpr int PP_TILE = PP_PAGE * PP_D * 2;  // 32 KB
constexpr int PP_STAGES = 3;
constexpr int PP_RING = 16;                  // unit ids fetched ahead of the compute cursor

__device__ __forceinline__ uint32_t pp_sw128(int row, int col_elem) {
  const int unit = (col_elem >> 3) ^ (row & 7);
  return row * 128 + unit * 16 + (col_elem & 7) * 2;
}

__device__ __forceinline__ void cp_async_16(uint32_t smem_dst, const void* gsrc) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_dst), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

template <int NCOL>
struct PpCfg {
  static constexpr int NPAD = NCOL <= 16 ? 16 : 32;                 // MMA N
  static constexpr int QBYTES = 2 * NPAD * 128;                      // [2 K-chunks][NPAD rows][64] bf16
  static constexpr int SMEM = PP_STAGES * 2 * PP_TILE + 3 * QBYTES + 2 * 4 * NCOL * 4 + 512 + 1024;
};

struct PpUnit {        // one (item, kv head, split)
  int b0, hk, sp, ncols, n_keys, page0, blk_begin, nb;
};

__device__ __forceinline__ PpUnit pp_decode(int u, const int* item_first, const int* item_size, const int* item_page0,
                                            const int* item_keys, int Hkv, int nsplit, int rep, int ncol_max) {
  PpUnit x;
  const int sp = u % nsplit, t = u / nsplit;
  x.sp = sp;
  x.hk = t % Hkv;
  const int w = t / Hkv;
  const int gsize = item_size[w];
  x.b0 = item_first[w];
  x.page0 = item_page0[w];
  x.n_keys = gsize > 0 ? item_keys[w] : 0;
  x.ncols = min(max(gsize, 0) * rep, ncol_max);
  const int n_blocks = (x.n_keys + PP_PAGE - 1) / PP_PAGE;
  const int per = (n_blocks + nsplit - 1) / nsplit;
  x.blk_begin = sp * per;
  x.nb = max(0, min(n_blocks, x.blk_begin + per) - x.blk_begin);
  if (gsize <= 0) x.nb = -1;      // inactive item: nothing to compute, nothing to write
  return x;
}

// items as in paged_decode_items_kernel; total = n_items * Hkv * nsplit work units. work_counter must be 0 at launch.
// out != nullptr (only with nslots == 1 and single-sequence items): write the normalised bf16 result directly.
template <int NCOL>
__global__ void __launch_bounds__(128, 1)
paged_decode_persist_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                            const __nv_bfloat16* __restrict__ q, long long q_row_stride,
                            const int* __restrict__ block_table, int max_pages, const int* __restrict__ item_first,
                            const int* __restrict__ item_size, const int* __restrict__ item_page0,
                            const int* __restrict__ item_keys, int n_items, int slot0, int neutral_from, int neutral_n,
                            float* __restrict__ part_o, float* __restrict__ part_ml, __nv_bfloat16* __restrict__ out,
                            int Hq, int Hkv, int nsplit, int nslots, float scale_log2, unsigned int* work_counter,
                            int* status) {
  using Cfg = PpCfg<NCOL>;
  constexpr int NPAD = Cfg::NPAD;
  grid_launch_dependents();
  const int rep = Hq / Hkv;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int total = n_items * Hkv * nsplit;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sKV = smem;                                   // [stage][K 32K | V 32K]
  uint8_t* sQ = smem + PP_STAGES * 2 * PP_TILE;          // two query buffers, used in turn by successive units
  uint8_t* sP = sQ + 2 * Cfg::QBYTES;
  float* red = reinterpret_cast<float*>(sP + Cfg::QBYTES);    // [2][4 warps][NCOL]
  uint8_t* tail = reinterpret_cast<uint8_t*>(red) + 2 * 4 * NCOL * 4;
  uint64_t* full = reinterpret_cast<uint64_t*>(tail);    // [PP_STAGES]
  uint64_t* bar_mma = full + PP_STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_mma + 1);
  int* ring = reinterpret_cast<int*>(tmem_slot + 2);     // [PP_RING] unit ids in processing order, -1 = no more work

  if (tid == 0) {
    for (int s = 0; s < PP_STAGES; ++s) mbar_init(&full[s], 1);
    mbar_init(bar_mma, 1);
    mbar_fence_init();
  }
  if (warp == 0) {
    tmem_alloc(tmem_slot, 2 * NPAD);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tS = tmem_base + (static_cast<uint32_t>(warp * 32) << 16);
  const uint32_t tO = tS + NPAD;
  constexpr uint32_t idesc_s = umma_idesc(128, NPAD, 0, 0);
  constexpr uint32_t idesc_o = umma_idesc(128, NPAD, 1, 0);

  // ---- thread 0: unit fetching and the load cursor (these variables are meaningful in thread 0 only)
  int rw = 0;                    // units fetched into the ring so far
  int rl = 0;                    // ring index of the unit the load cursor is in
  int lblk = 0, l_nb = 0, l_hk = 0;
  const int* l_bt = block_table;
  bool l_open = false;           // the load cursor has a unit with blocks left
  bool l_end = false;            // the load cursor has seen the end marker
  long long g_issue = 0;         // K|V blocks whose loads were issued (all units of this CTA)
  long long g_done = 0;          // blocks whose stage may be overwritten (their P*V product has completed)

  // Unit ids come from an atomic counter. The atomic's round trip to L2 is hidden by splitting the fetch: the request
  // is made at the start of a unit and its result is first touched (written into the ring) one unit later.
  unsigned int pend = 0;
  bool has_pend = false;
  auto fetch_begin = [&]() {     // thread 0
    pend = atomicAdd(work_counter, 1u);
    has_pend = true;
  };
  auto fetch_commit = [&]() {    // thread 0
    ring[rw % PP_RING] = pend < (unsigned int)total ? (int)pend : -1;
    ++rw;
    has_pend = false;
  };
  auto fetch_unit = [&]() {      // thread 0: request and use at once (start-up, or the load cursor ran out of known units)
    if (!has_pend) fetch_begin();
    fetch_commit();
  };
  auto advance_loads = [&](int rr) {   // thread 0: issue loads while a stage is free; rr = compute cursor's ring index
    while (!l_end && g_issue < g_done + PP_STAGES) {
      if (!l_open) {
        if (rl >= rw) {
          if (rw - rr >= PP_RING - 1) break;     // ring full: wait for the compute cursor
          fetch_unit();
        }
        const int u = ring[rl % PP_RING];
        if (u < 0) {
          l_end = true;
          break;
        }
        const PpUnit x = pp_decode(u, item_first, item_size, item_page0, item_keys, Hkv, nsplit, rep, NCOL);
        if (x.nb <= 0) {
          ++rl;
          continue;
        }
        l_bt = block_table + (long long)x.b0 * max_pages + x.page0 + x.blk_begin;
        l_nb = x.nb;
        l_hk = x.hk;
        lblk = 0;
        l_open = true;
      }
      const int s = (int)(g_issue % PP_STAGES);
      const int page = l_bt[lblk];
      const int row0 = (page * Hkv + l_hk) * PP_PAGE;
      uint8_t* k = sKV + s * 2 * PP_TILE;
      mbar_expect_tx(&full[s], 2 * PP_TILE);
      tma_load_2d(k, &tmK, &full[s], 0, row0);
      tma_load_2d(k + 16384, &tmK, &full[s], 64, row0);
      tma_load_2d(k + PP_TILE, &tmV, &full[s], 0, row0);
      tma_load_2d(k + PP_TILE + 16384, &tmV, &full[s], 64, row0);
      ++g_issue;
      if (++lblk >= l_nb) {
        l_open = false;
        ++rl;
      }
    }
  };
  // query rows of a unit -> sQ[buf] with cp.async (16-byte pieces keep the 128-byte swizzle's granularity)
  auto fetch_q = [&](const PpUnit& x, int buf) {
    const uint32_t base = smem_u32(sQ + buf * Cfg::QBYTES);
    for (int i = tid; i < x.ncols * 16; i += 128) {
      const int c = i >> 4, piece = i & 15;            // column (sequence, head) and 16-byte piece of its 128 dims
      const __nv_bfloat16* src = q + (long long)(x.b0 + c / rep) * q_row_stride + (long long)(x.hk * rep + c % rep) * PP_D + piece * 8;
      cp_async_16(base + (piece >> 3) * (NPAD * 128) + pp_sw128(c, (piece & 7) * 8), src);
    }
    cp_async_commit();
  };

  // zero both query buffers once: rows beyond a unit's columns must not hold NaN patterns
  for (int i = tid; i < 2 * Cfg::QBYTES / 16; i += 128) reinterpret_cast<uint4*>(sQ)[i] = make_uint4(0, 0, 0, 0);
  if (tid == 0) {
    fetch_unit();
    fetch_unit();
  }
  __syncthreads();

  bool ok = true;
  uint32_t ph = 0;          // bar_mma: one completion per block (after S) and one after a unit's last P*V
  long long g = 0;          // blocks consumed so far by this CTA (selects stage and parity)
  int rr = 0;               // compute cursor: ring index of the current unit
  int u_cur = ring[0];
  PpUnit cur;
  cur.nb = -1;
  if (u_cur >= 0) cur = pp_decode(u_cur, item_first, item_size, item_page0, item_keys, Hkv, nsplit, rep, NCOL);
  int qbuf = 0;             // query buffer the current unit reads
  int q_unit = -1;          // ring index of the unit whose query rows were last requested (into qbuf, or qbuf ^ 1 if it is rr + 1)

  while (u_cur >= 0) {
    // next unit id (thread 0 keeps the ring one ahead), and its query rows into the other buffer
    if (tid == 0) {
      if (has_pend) fetch_commit();
      while (rw < rr + 2) fetch_unit();
      if (rw - rr < PP_RING - 1) fetch_begin();          // the unit after next: asked for now, looked at one unit from now
      advance_loads(rr);
    }
    __syncthreads();
    const int u_next = ring[(rr + 1) % PP_RING];
    PpUnit nxt;
    nxt.nb = -1;
    if (u_next >= 0) nxt = pp_decode(u_next, item_first, item_size, item_page0, item_keys, Hkv, nsplit, rep, NCOL);

    if (cur.nb >= 0) {
      const int ncols = cur.ncols;
      // slots this item never fills for its sequences: no shared prefix -> neutral prefix slots
      if (neutral_n > 0 && cur.page0 == 0 && cur.sp == 0) {
        for (int i = tid; i < ncols * neutral_n; i += 128) {
          const int c = i / neutral_n, sl = i % neutral_n;
          const long long idx = ((long long)(cur.b0 + c / rep) * Hq + cur.hk * rep + c % rep) * nslots + neutral_from + sl;
          part_ml[idx * 2] = -1e30f;
          part_ml[idx * 2 + 1] = 0.f;
        }
      }
      if (cur.nb == 0) {
        if (out != nullptr) {                      // a row without keys (padding of a batch bucket): zeros
          for (int c = 0; c < ncols; ++c)
            out[((long long)(cur.b0 + c / rep) * Hq + cur.hk * rep + c % rep) * PP_D + tid] = __float2bfloat16(0.f);
        } else if (tid < ncols) {
          const long long idx = ((long long)(cur.b0 + tid / rep) * Hq + cur.hk * rep + tid % rep) * nslots + slot0 + cur.sp;
          part_ml[idx * 2] = -1e30f;
          part_ml[idx * 2 + 1] = 0.f;
        }
      } else if (ok) {
        // the unit's query rows were requested while the previous unit computed; if that unit did no work (or this is
        // the first one) they are requested now
        if (q_unit != rr) {
          fetch_q(cur, qbuf);
          q_unit = rr;
        }
        cp_async_wait_all();
        fence_async_shared();
        tc_fence_before();
        __syncthreads();
        tc_fence_after();
        if (nxt.nb > 0) {
          fetch_q(nxt, qbuf ^ 1);
          q_unit = rr + 1;
        }
        const uint32_t qaddr = smem_u32(sQ + qbuf * Cfg::QBYTES);

        float m_run[NCOL], l_thr[NCOL];
#pragma unroll
        for (int c = 0; c < NCOL; ++c) {
          m_run[c] = -1e30f;
          l_thr[c] = 0.f;
        }
        const int nb = cur.nb;
        for (int i = 0; i < nb; ++i, ++g) {
          const int s = (int)(g % PP_STAGES);
          const uint32_t kaddr = smem_u32(sKV + s * 2 * PP_TILE);
          if (tid == 0 && ok) {
            if (!mbar_wait(&full[s], (uint32_t)((g / PP_STAGES) & 1))) {
              report_error(status, AXB_ERR_WAIT_FULL);
              ok = false;
            }
            tc_fence_after();
            if (ok) {
#pragma unroll
              for (int ks = 0; ks < 8; ++ks) {
                umma_f16_ss(tmem_base, umma_smem_desc(kaddr + (ks >> 2) * 16384 + (ks & 3) * 32, 16, 1024),
                            umma_smem_desc(qaddr + (ks >> 2) * (NPAD * 128) + (ks & 3) * 32, 16, 1024), idesc_s, ks != 0);
              }
              tc_commit(bar_mma);   // also covers the P*V product of the previous block
            }
          }
          // every thread learns whether thread 0 gave up (uniform control flow from here on)
          ok = __syncthreads_and(ok ? 1 : 0) != 0;
          if (!ok) break;
          if (!mbar_wait(bar_mma, ph)) {
            report_error(status, AXB_ERR_WAIT_TMEM_FULL);
            ok = false;
          }
          ph ^= 1;
          tc_fence_after();
          // the stage of the previous block is free now: keep the ring full, across the unit boundary if need be
          if (tid == 0 && ok) {
            g_done = g;
            advance_loads(rr);
          }

          uint32_t sv[NPAD];
          tmem_ld_32x16(tS, sv);
          if (NPAD == 32) tmem_ld_32x16(tS + 16, sv + 16);
          tmem_ld_wait();
          const int kpos = (cur.blk_begin + i) * PP_PAGE + tid;
          const bool valid = kpos < cur.n_keys;
          float sc[NCOL];
#pragma unroll
          for (int c = 0; c < NCOL; ++c) {
            sc[c] = (valid && c < ncols) ? __uint_as_float(sv[c]) * scale_log2 : -INFINITY;
            const float wm = warp_max_redux(sc[c]);
            if (lane == 0) red[((i & 1) * 4 + warp) * NCOL + c] = wm;
          }
          ok = __syncthreads_and(ok ? 1 : 0) != 0;
          if (!ok) break;
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
              *reinterpret_cast<__nv_bfloat16*>(sP + (tid >> 6) * (NPAD * 128) + pp_sw128(c, tid & 63)) = __float2bfloat16(p);
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
          if (tid == 0) {
            tc_fence_after();
            const uint32_t vaddr = kaddr + PP_TILE, paddr = smem_u32(sP);
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
        if (ok) {
          if (!mbar_wait(bar_mma, ph)) {
            report_error(status, AXB_ERR_WAIT_TMEM_FULL);
            ok = false;
          }
          ph ^= 1;
          tc_fence_after();
          if (tid == 0) {
            g_done = g;                 // the unit's last stage is free as well
            advance_loads(rr);
          }
        }
        ok = __syncthreads_and(ok ? 1 : 0) != 0;
        if (ok) {
          // ---- unit epilogue: un-normalised partials. l per column: reduce the per-thread sums over the CTA.
          float l_tot[NCOL];
#pragma unroll
          for (int c = 0; c < NCOL; ++c) {
            const float ws = warp_sum(l_thr[c]);
            if (lane == 0) red[warp * NCOL + c] = ws;
          }
          __syncthreads();
#pragma unroll
          for (int c = 0; c < NCOL; ++c) l_tot[c] = red[c] + red[NCOL + c] + red[2 * NCOL + c] + red[3 * NCOL + c];
          uint32_t o[NPAD];
          tmem_ld_32x16(tO, o);
          if (NPAD == 32) tmem_ld_32x16(tO + 16, o + 16);
          tmem_ld_wait();
#pragma unroll
          for (int c = 0; c < NCOL; ++c) {
            if (c < ncols) {
              const long long bh = (long long)(cur.b0 + c / rep) * Hq + cur.hk * rep + c % rep;
              if (out != nullptr) {
                out[bh * PP_D + tid] = __float2bfloat16(l_tot[c] > 0.f ? __uint_as_float(o[c]) / l_tot[c] : 0.f);
              } else {
                const long long idx = bh * nslots + slot0 + cur.sp;
                part_o[idx * PP_D + tid] = __uint_as_float(o[c]);
                if (tid == 0) {
                  part_ml[idx * 2] = m_run[c];
                  part_ml[idx * 2 + 1] = l_tot[c];
                }
              }
            }
          }
          tc_fence_before();      // the next unit's first S product overwrites the accumulators read above
          __syncthreads();
          tc_fence_after();
          if (q_unit == rr + 1) qbuf ^= 1;      // the next unit's rows sit in the other buffer
        }
      }
    }
    if (!ok) break;
    // move on
    ++rr;
    u_cur = u_next;
    cur = nxt;
  }

  // ---- shut down. After an error loads may still be in flight: wait for them (bounded) before the memory goes away.
  cp_async_wait_all();
  if (!ok && tid == 0) {
    for (long long b = g; b < g_issue; ++b) mbar_wait(&full[b % PP_STAGES], (uint32_t)((b / PP_STAGES) & 1));
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 2 * NPAD);
  }
}

// out[b][h][:] = sum_s O_s 2^(m_s - M) / sum_s l_s 2^(m_s - M) over the nslots partial slots of (b, h)
__global__ void pp_merge_slots_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
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
    acc += part_o[(bh * nslots + s) * PP_D + d] * w;
    l += ls * w;
  }
  out[bh * PP_D + d] = __float2bfloat16(l > 0.f ? acc / l : 0.f);
}

}  // namespace axb

using namespace axb;

namespace {
int persist_grid(int total) {
  const int sms = sm_count();
  return total < sms ? total : sms;
}
template <int NCOL>
int set_attr() {
  static bool done = false;
  if (!done) {
    if (cudaFuncSetAttribute(paged_decode_persist_kernel<NCOL>, cudaFuncAttributeMaxDynamicSharedMemorySize, PpCfg<NCOL>::SMEM) !=
        cudaSuccess)
      return AXB_LAUNCH_CUDA_ERROR;
    done = true;
  }
  return AXB_LAUNCH_OK;
}
}  // namespace

// Same arguments as axb_paged_decode_shared plus `counters`: two 32-bit words the launcher zeroes (stream-ordered)
// and the kernels use as work counters.
extern "C" int axb_paged_decode_shared_persist(const void* q, long long q_row_stride, const void* kcache, const void* vcache,
                                               int num_pages, const int* block_table, int max_pages, const int* seq_first,
                                               const int* seq_one, const int* seq_page0, const int* seq_keys,
                                               const int* grp_first, const int* grp_size, const int* grp_zero,
                                               const int* grp_keys, int n_groups, void* out, int B, int Hq, int Hkv, int D,
                                               float softmax_scale, int nsplit, int nsplit_p, void* scratch,
                                               unsigned int* counters, int* status, void* stream) {
  if (D != PP_D || B <= 0 || n_groups < 0 || Hq % Hkv != 0 || Hq / Hkv > 8 || nsplit < 1 || nsplit_p < 1 || scratch == nullptr ||
      counters == nullptr)
    return AXB_LAUNCH_BAD_ARG;
  cudaStream_t s = (cudaStream_t)stream;
  CUtensorMap tmK, tmV;
  const unsigned long long rows = (unsigned long long)num_pages * Hkv * PP_PAGE;
  int rc = make_tmap_2d(&tmK, kcache, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, PP_D, rows, PP_D * 2, 64, PP_PAGE, true);
  if (rc) return rc;
  rc = make_tmap_2d(&tmV, vcache, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, PP_D, rows, PP_D * 2, 64, PP_PAGE, true);
  if (rc) return rc;
  if ((rc = set_attr<8>()) || (rc = set_attr<32>())) return rc;
  if (cudaMemsetAsync(counters, 0, 2 * sizeof(unsigned int), s) != cudaSuccess) return AXB_LAUNCH_CUDA_ERROR;
  const bool direct = n_groups == 0 && nsplit == 1;          // no prefix items, one split: the result needs no merge
  const int nslots = n_groups == 0 ? nsplit : nsplit + nsplit_p;
  float* part_o = reinterpret_cast<float*>(scratch);
  float* part_ml = part_o + (long long)B * Hq * nslots * PP_D;
  const float sl2 = softmax_scale * 1.4426950408889634f;
  // suffix items: one sequence each, slots [0, nsplit); they neutralise the prefix slots of unshared sequences
  const int total_s = B * Hkv * nsplit;
  paged_decode_persist_kernel<8><<<persist_grid(total_s), 128, PpCfg<8>::SMEM, s>>>(
      tmK, tmV, (const __nv_bfloat16*)q, q_row_stride, block_table, max_pages, seq_first, seq_one, seq_page0, seq_keys, B,
      0, nsplit, n_groups == 0 ? 0 : nsplit_p, part_o, part_ml, direct ? (__nv_bfloat16*)out : nullptr, Hq, Hkv, nsplit, nslots,
      sl2, counters, status);
  rc = check_launch();
  if (rc || direct) return rc;
  if (n_groups > 0) {
    // prefix items: one group each, slots [nsplit, nsplit + nsplit_p)
    const int total_p = n_groups * Hkv * nsplit_p;
    paged_decode_persist_kernel<32><<<persist_grid(total_p), 128, PpCfg<32>::SMEM, s>>>(
        tmK, tmV, (const __nv_bfloat16*)q, q_row_stride, block_table, max_pages, grp_first, grp_size, grp_zero, grp_keys,
        n_groups, nsplit, 0, 0, part_o, part_ml, nullptr, Hq, Hkv, nsplit_p, nslots, sl2, counters + 1, status);
    rc = check_launch();
    if (rc) return rc;
  }
  pp_merge_slots_kernel<<<B * Hq, PP_D, 0, s>>>(part_o, part_ml, (__nv_bfloat16*)out, nslots);
  return check_launch();
}
