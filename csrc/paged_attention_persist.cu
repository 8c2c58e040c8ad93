// Persistent, warp-specialised form of the item-based paged decode attention (paged_attention_shared.cu).
//
// The item kernels launch one CTA per (item, kv head, key split) and run every step of a key block - tile wait,
// S product, softmax, P*V product, next loads - one after the other on the same 128 threads. Counters of that
// kernel show ~4000 cycles per 64 KB block with most issue slots lost at CTA-wide barriers, i.e. ~0.7 of the HBM
// rate, and with short items (the private tail of a sample after its shared prompt) the per-CTA start-up costs as
// much as the keys themselves.
//
// Here ONE CTA per SM lives for the whole launch, pulls work units (item, kv head, split) from an atomic counter
// and splits the work over three roles that only meet at mbarriers:
//
//   producer warp   fetches unit ids, loads each unit's query rows and its K / V tiles by TMA into a ring of six
//                   32 KB slots (K0 V0 K1 V1 ...), running ahead of the consumers by up to six tiles - across unit
//                   boundaries, so the pipeline never drains between units;
//   MMA warp        one thread issues S^T = K_tile Q^T (tcgen05, N = query columns) for block g+1 BEFORE the
//                   O^T += V_tile^T P^T product of block g, so the tensor core always has the next scores ready
//                   when the softmax threads finish a block; tcgen05.commit releases the tile slots;
//   softmax threads 128 threads, thread t owns key t of the block and output dimension t in the epilogue. The
//                   running maximum is raised lazily: a block first checks with one OR-reducing barrier whether
//                   any score exceeds the running maximum by more than 2^8; only then (the first block of a unit
//                   and rare later ones) are exact column maxima exchanged and the accumulator rescaled.
//
// TMEM holds two S accumulators (alternating by block) and two O accumulators (alternating by unit), shared
// memory two query buffers (by unit) and two P buffers (by block), so that no role waits for another one's
// previous step. Results are un-normalised partials per (sequence, head, slot) merged by pp_merge_slots_kernel,
// or the normalised bf16 output directly when there is one slot.
//
// Every wait is bounded; a wait that runs out records a status code and raises an abort flag that all roles
// poll; the producer then waits (bounded) for its loads in flight, TMEM is freed and the kernel returns.
#include "ptx.cuh"
#include "host_utils.h"

namespace axb {

constexpr int PP_D = 128;
constexpr int PP_PAGE = 128;
constexpr int PP_TILE = PP_PAGE * PP_D * 2;  // 32 KB: the K (or V) rows of one page and kv head
constexpr int PP_SLOTS = 6;                  // tile slots: K and V tiles of successive blocks alternate
constexpr int PP_RING = 16;                  // unit ids published ahead of the slowest consumer
constexpr int PP_THREADS = 192;              // 4 softmax warps + producer warp + MMA warp

__device__ __forceinline__ uint32_t pp_sw128(int row, int col_elem) {
  const int unit = (col_elem >> 3) ^ (row & 7);
  return row * 128 + unit * 16 + (col_elem & 7) * 2;
}
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// barrier 1 over the 128 softmax threads
__device__ __forceinline__ void softmax_bar_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }
__device__ __forceinline__ bool softmax_bar_or(bool p) {
  uint32_t r;
  asm volatile(
      "{\n\t"
      ".reg .pred p, q;\n\t"
      "setp.ne.b32 p, %1, 0;\n\t"
      "barrier.red.or.pred q, 1, 128, p;\n\t"
      "selp.u32 %0, 1, 0, q;\n\t"
      "}\n"
      : "=r"(r)
      : "r"((uint32_t)p)
      : "memory");
  return r != 0;
}

template <int NCOL>
struct PpCfg {
  static constexpr int NPAD = NCOL <= 16 ? 16 : 32;                 // MMA N
  static constexpr int QBYTES = 2 * NPAD * 128;                      // [2 K-chunks][NPAD rows][64] bf16
  static constexpr int TCOLS = 4 * NPAD;                             // S0 | S1 | O0 | O1
  static constexpr int SMEM = PP_SLOTS * PP_TILE + 4 * QBYTES + 2 * 4 * NCOL * 4 + 1024 + 1024;
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
// tmQ: the query rows as a 3-D tensor [sequence][head][128] with box (64, rep, sequences per item).
// out != nullptr (only with nslots == 1 and single-sequence items): write the normalised bf16 result directly.
template <int NCOL>
__global__ void __launch_bounds__(PP_THREADS, 1)
paged_decode_persist_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                            const __grid_constant__ CUtensorMap tmQ, int q_box_bytes,
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
  uint8_t* sT = smem;                                    // [slot] 32 KB tiles; tile 2g = K of block g, 2g+1 = V of block g
  uint8_t* sQ = smem + PP_SLOTS * PP_TILE;               // two query buffers, by unit
  uint8_t* sP = sQ + 2 * Cfg::QBYTES;                    // two probability buffers, by block
  float* red = reinterpret_cast<float*>(sP + 2 * Cfg::QBYTES);   // [4 warps][NCOL] column maxima, then [4][NCOL] row sums
  uint8_t* tail = reinterpret_cast<uint8_t*>(red) + 2 * 4 * NCOL * 4;
  uint64_t* full = reinterpret_cast<uint64_t*>(tail);    // [PP_SLOTS] tile landed
  uint64_t* empty = full + PP_SLOTS;                     // [PP_SLOTS] the product that read the tile has completed
  uint64_t* q_full = empty + PP_SLOTS;                   // [2] query rows landed
  uint64_t* q_empty = q_full + 2;                        // [2] the unit's last S product has completed
  uint64_t* bar_s = q_empty + 2;                         // [2] S of a block has completed
  uint64_t* p_ready = bar_s + 2;                         // [2] 128 arrivals: P written (and O rescaled) for a block
  uint64_t* bar_pv = p_ready + 2;                        // [2] P*V of an even / odd block has completed
  uint64_t* o_free = bar_pv + 2;                         // [2] 128 arrivals: the unit's accumulator has been read
  uint64_t* ring_full = o_free + 2;                      // [PP_RING] unit id published
  uint64_t* ring_empty = ring_full + PP_RING;            // [PP_RING] 128 arrivals: the softmax threads are done with the unit
  int* ring = reinterpret_cast<int*>(ring_empty + PP_RING);   // [PP_RING] unit ids in processing order, -1 = no more work
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(ring + PP_RING);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  if (tid == 0) {
    for (int s = 0; s < PP_SLOTS; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int k = 0; k < 2; ++k) {
      mbar_init(&q_full[k], 1);
      mbar_init(&q_empty[k], 1);
      mbar_init(&bar_s[k], 1);
      mbar_init(&p_ready[k], 128);
      mbar_init(&o_free[k], 128);
      mbar_init(&bar_pv[k], 1);
    }
    for (int k = 0; k < PP_RING; ++k) {
      mbar_init(&ring_full[k], 1);
      mbar_init(&ring_empty[k], 128);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 5) {
    tmem_alloc(tmem_slot, Cfg::TCOLS);
    tmem_relinquish();
  }
  // query and probability buffers start as zeros: rows beyond a unit's columns must not hold NaN patterns
  for (int i = tid; i < 4 * Cfg::QBYTES / 16; i += PP_THREADS) reinterpret_cast<uint4*>(sQ)[i] = make_uint4(0, 0, 0, 0);
  fence_async_shared();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  auto give_up = [&](int code) {
    report_error(status, code);
    *abort_flag = 1;
  };

  if (warp == 4) {
    // ================================================================== producer: unit ids, query rows, K / V tiles
    long long t = 0;           // tiles issued
    int nq = 0;                // units with blocks so far (selects the query buffer)
    bool ok = true;
    for (int n = 0; ok; ++n) {
      int u = -1;
      if (lane == 0) {
        if (n >= PP_RING && !mbar_wait(&ring_empty[n % PP_RING], (uint32_t)(((n / PP_RING) - 1) & 1))) {
          give_up(AXB_ERR_WAIT_EMPTY);
          ok = false;
        }
        if (ok) {
          const unsigned int v = atomicAdd(work_counter, 1u);
          u = v < (unsigned int)total ? (int)v : -1;
        }
        ring[n % PP_RING] = u;
        mbar_arrive(&ring_full[n % PP_RING]);       // release: the id is visible to whoever passes the barrier
      }
      u = __shfl_sync(0xffffffffu, u, 0);
      ok = __shfl_sync(0xffffffffu, (int)(ok && *abort_flag == 0), 0) != 0;      // lane 0 decides for the warp
      if (u < 0 || !ok) break;
      const PpUnit x = pp_decode(u, item_first, item_size, item_page0, item_keys, Hkv, nsplit, rep, NCOL);
      if (x.nb <= 0) continue;
      if (lane == 0) {
        const int qb = nq & 1;
        if (nq >= 2 && !mbar_wait(&q_empty[qb], (uint32_t)(((nq >> 1) - 1) & 1))) {
          give_up(AXB_ERR_WAIT_EMPTY);
          ok = false;
        } else {
          mbar_expect_tx(&q_full[qb], 2 * q_box_bytes);
          tma_load_3d(sQ + qb * Cfg::QBYTES, &tmQ, &q_full[qb], 0, x.hk * rep, x.b0);
          tma_load_3d(sQ + qb * Cfg::QBYTES + NPAD * 128, &tmQ, &q_full[qb], 64, x.hk * rep, x.b0);
        }
      }
      ++nq;
      const int* bt = block_table + (long long)x.b0 * max_pages + x.page0 + x.blk_begin;
      for (int blk0 = 0; blk0 < x.nb && ok; blk0 += 32) {
        const int mine = blk0 + lane < x.nb ? bt[blk0 + lane] : 0;       // 32 page ids with one coalesced load
        const int cnt = min(32, x.nb - blk0);
        for (int j = 0; j < cnt; ++j) {
          const int page = __shfl_sync(0xffffffffu, mine, j);
          if (lane == 0 && ok) {
            const int row0 = (page * Hkv + x.hk) * PP_PAGE;
            for (int half = 0; half < 2 && ok; ++half, ++t) {
              const int s = (int)(t % PP_SLOTS);
              if (t >= PP_SLOTS && !mbar_wait(&empty[s], (uint32_t)(((t / PP_SLOTS) - 1) & 1))) {
                give_up(AXB_ERR_WAIT_EMPTY);
                ok = false;
                break;
              }
              uint8_t* dst = sT + s * PP_TILE;
              mbar_expect_tx(&full[s], PP_TILE);
              tma_load_2d(dst, half == 0 ? &tmK : &tmV, &full[s], 0, row0);
              tma_load_2d(dst + 16384, half == 0 ? &tmK : &tmV, &full[s], 64, row0);
            }
          }
        }
        ok = __shfl_sync(0xffffffffu, (int)(ok && *abort_flag == 0), 0) != 0;
      }
    }
    // after an error loads may still be in flight: wait (bounded) for the latest use of every slot and query buffer
    if (lane == 0 && *abort_flag != 0) {
      for (long long b = t > PP_SLOTS ? t - PP_SLOTS : 0; b < t; ++b)
        mbar_wait(&full[b % PP_SLOTS], (uint32_t)((b / PP_SLOTS) & 1));
      for (int b = nq > 2 ? nq - 2 : 0; b < nq; ++b) mbar_wait(&q_full[b & 1], (uint32_t)((b >> 1) & 1));
    }
  } else if (warp == 5) {
    // ================================================================== MMA issuer (one thread)
    if (lane == 0) {
      constexpr uint32_t idesc_s = umma_idesc(128, NPAD, 0, 0);
      constexpr uint32_t idesc_o = umma_idesc(128, NPAD, 1, 0);
      bool ok = true;
      int n = 0;                 // ring position of the S cursor
      int nq = 0;                // units with blocks the S cursor has entered
      long long g = 0;           // blocks whose S product has been issued
      PpUnit x;
      x.nb = 0;
      int i = 0;                 // S cursor: next block of x
      bool more = true;
      // the block whose P*V product is still to be issued (always the one before the S cursor)
      bool pend = false, pend_first = false;
      long long pend_g = 0;
      int pend_ob = 0, pend_nq = 0;
      auto issue_pv = [&]() {
        const int s = (int)((2 * pend_g + 1) % PP_SLOTS);
        if (!mbar_wait(&p_ready[pend_g & 1], (uint32_t)((pend_g >> 1) & 1)) ||
            !mbar_wait(&full[s], (uint32_t)(((2 * pend_g + 1) / PP_SLOTS) & 1)) ||
            (pend_first && pend_nq >= 2 && !mbar_wait(&o_free[pend_ob], (uint32_t)(((pend_nq >> 1) - 1) & 1)))) {
          give_up(AXB_ERR_WAIT_TMEM_EMPTY);
          ok = false;
          return;
        }
        tc_fence_after();
        const uint32_t vaddr = smem_u32(sT + s * PP_TILE), paddr = smem_u32(sP + (pend_g & 1) * Cfg::QBYTES);
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          umma_f16_ss(tmem_base + (2 + pend_ob) * NPAD, umma_smem_desc(vaddr + ks * 2048, 16384, 1024),
                      umma_smem_desc(paddr + (ks >> 2) * (NPAD * 128) + (ks & 3) * 32, 16, 1024), idesc_o,
                      (!pend_first || ks != 0) ? 1u : 0u);
        }
        tc_commit(&empty[s]);
        tc_commit(&bar_pv[pend_g & 1]);
      };
      while (ok && more) {
        // ---- move the S cursor to the next block (entering the next unit with blocks if need be)
        while (i >= x.nb) {
          // Never block on an unpublished unit with a product still owed: the producer may be waiting for the softmax
          // threads to finish the unit that needs it (a run of sixteen units without blocks closes that cycle).
          if (pend && !mbar_try_wait(&ring_full[n % PP_RING], (uint32_t)((n / PP_RING) & 1))) {
            issue_pv();
            pend = false;
            if (!ok) break;
          }
          if (!mbar_wait(&ring_full[n % PP_RING], (uint32_t)((n / PP_RING) & 1))) {
            give_up(AXB_ERR_WAIT_FULL);
            ok = false;
            break;
          }
          const int u = ring[n % PP_RING];
          ++n;
          if (u < 0) {
            more = false;
            break;
          }
          x = pp_decode(u, item_first, item_size, item_page0, item_keys, Hkv, nsplit, rep, NCOL);
          i = 0;
          if (x.nb > 0) {
            if (!mbar_wait(&q_full[nq & 1], (uint32_t)((nq >> 1) & 1))) {
              give_up(AXB_ERR_WAIT_FULL);
              ok = false;
              break;
            }
            ++nq;
          }
        }
        if (!ok || !more || *abort_flag != 0) break;
        // ---- S of block g: its accumulator was read by the softmax two blocks back, whose P this thread has waited for
        {
          const int s = (int)((2 * g) % PP_SLOTS);
          if (!mbar_wait(&full[s], (uint32_t)(((2 * g) / PP_SLOTS) & 1))) {
            give_up(AXB_ERR_WAIT_FULL);
            ok = false;
            break;
          }
          tc_fence_after();
          const int qb = (nq - 1) & 1;
          const uint32_t kaddr = smem_u32(sT + s * PP_TILE), qaddr = smem_u32(sQ + qb * Cfg::QBYTES);
#pragma unroll
          for (int ks = 0; ks < 8; ++ks) {
            umma_f16_ss(tmem_base + (uint32_t)(g & 1) * NPAD, umma_smem_desc(kaddr + (ks >> 2) * 16384 + (ks & 3) * 32, 16, 1024),
                        umma_smem_desc(qaddr + (ks >> 2) * (NPAD * 128) + (ks & 3) * 32, 16, 1024), idesc_s, ks != 0);
          }
          tc_commit(&bar_s[g & 1]);
          tc_commit(&empty[s]);
          if (i == x.nb - 1) tc_commit(&q_empty[qb]);
        }
        // ---- P*V of the block before it
        if (pend) issue_pv();
        pend = true;
        pend_g = g;
        pend_first = i == 0;
        pend_nq = nq - 1;
        pend_ob = (nq - 1) & 1;
        ++g;
        ++i;
      }
      if (ok && pend && *abort_flag == 0) issue_pv();
    }
  } else {
    // ================================================================== softmax and epilogue (128 threads; thread = key / dim)
    const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(warp * 32) << 16);
    // `fail` is this thread's own finding (a wait ran out); the threads only leave their loops together, on `quit`,
    // which is always the result of an OR-reducing barrier
    bool fail = false, quit = false;
    int nq = 0;
    long long g = 0;
    // this thread's byte offset inside a P buffer for column 0; column c adds c * 128 and flips the 16-byte unit by c & 7
    const int pcol = tid & 63;
    uint8_t* const pbase = sP + (tid >> 6) * (NPAD * 128);
    for (int n = 0; !quit; ++n) {
      if (!mbar_wait(&ring_full[n % PP_RING], (uint32_t)((n / PP_RING) & 1))) {
        give_up(AXB_ERR_WAIT_FULL);
        fail = true;
      }
      if (softmax_bar_or(fail)) break;
      const int u = ring[n % PP_RING];
      if (u < 0) break;
      const PpUnit cur = pp_decode(u, item_first, item_size, item_page0, item_keys, Hkv, nsplit, rep, NCOL);
      if (cur.nb >= 0) {
        const int ncols = cur.ncols;
        // slots this item never fills for its sequences: no shared prefix -> neutral prefix slots
        if (neutral_n > 0 && cur.page0 == 0 && cur.sp == 0) {
          for (int k = tid; k < ncols * neutral_n; k += 128) {
            const int c = k / neutral_n, sl = k % neutral_n;
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
        } else {
          const uint32_t tO = lane_base + (2 + (nq & 1)) * NPAD;
          float m_run[NCOL], l_thr[NCOL];
#pragma unroll
          for (int c = 0; c < NCOL; ++c) {
            m_run[c] = -1e30f;
            l_thr[c] = 0.f;
          }
          const int nb = cur.nb;
          for (int i = 0; i < nb; ++i, ++g) {
            if (!mbar_wait(&bar_s[g & 1], (uint32_t)((g >> 1) & 1))) {
              give_up(AXB_ERR_WAIT_TMEM_FULL);
              fail = true;
            }
            tc_fence_after();
            uint32_t sv[NPAD];
            const uint32_t tSg = lane_base + (uint32_t)(g & 1) * NPAD;
            tmem_ld_32x16(tSg, sv);
            if (NPAD == 32) tmem_ld_32x16(tSg + 16, sv + 16);
            tmem_ld_wait();
            const bool valid = (cur.blk_begin + i) * PP_PAGE + tid < cur.n_keys;
            float sc[NCOL];
            bool over = false;
#pragma unroll
            for (int c = 0; c < NCOL; ++c) {
              sc[c] = (valid && c < ncols) ? __uint_as_float(sv[c]) * scale_log2 : -INFINITY;
              over |= sc[c] > m_run[c] + 8.f;
            }
            // one barrier tells every thread whether any score of the block is more than 2^8 above its column's running
            // maximum, and whether anyone gave up (uniform control flow from here on)
            const bool slow = softmax_bar_or(over || fail || *abort_flag != 0);
            if (slow) {
              quit = softmax_bar_or(fail || *abort_flag != 0);
              if (quit) break;
              // exact column maxima over the 128 keys; raise the running maximum where the block exceeds it by > 2^8
#pragma unroll
              for (int c = 0; c < NCOL; ++c) {
                const float wm = warp_max_redux(sc[c]);
                if (lane == 0) red[warp * NCOL + c] = wm;
              }
              softmax_bar_sync();
              bool changed = false;
              float alpha[NCOL];
#pragma unroll
              for (int c = 0; c < NCOL; ++c) {
                const float bm = fmaxf(fmaxf(red[c], red[NCOL + c]), fmaxf(red[2 * NCOL + c], red[3 * NCOL + c]));
                const bool raise = bm > m_run[c] + 8.f;
                const float mn = raise ? bm : m_run[c];
                alpha[c] = raise ? ex2_approx(m_run[c] - mn) : 1.f;
                changed |= raise;
                m_run[c] = mn;
                l_thr[c] *= alpha[c];
              }
              if (i > 0 && changed) {  // uniform: m_run is identical in every thread
                // the accumulator holds the products up to the previous block: wait for that one, then rescale
                if (!mbar_wait(&bar_pv[(g - 1) & 1], (uint32_t)(((g - 1) >> 1) & 1))) {
                  give_up(AXB_ERR_WAIT_TMEM_FULL);
                  fail = true;
                }
                tc_fence_after();
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
            }
            // probabilities: the buffer of this parity was read by the product two blocks back, which completed before
            // this block's S product did (the tensor core runs one CTA's products in issue order)
            uint8_t* const pb = pbase + (g & 1) * Cfg::QBYTES;
#pragma unroll
            for (int c = 0; c < NCOL; ++c) {
              const float p = ex2_approx(sc[c] - m_run[c]);
              l_thr[c] += p;
              if (c < ncols) *reinterpret_cast<__nv_bfloat16*>(pb + pp_sw128(c, pcol)) = __float2bfloat16(p);
            }
            fence_async_shared();
            tc_fence_before();
            mbar_arrive(&p_ready[g & 1]);
          }
          if (quit) break;
          // ---- unit epilogue: wait for the last product, then un-normalised partials (or the normalised result)
          // (one barrier per block parity: the products two blocks back are known to be complete, the one two blocks
          // ahead cannot have been issued, so the phase parity is unambiguous although most blocks never wait here)
          if (!mbar_wait(&bar_pv[(g - 1) & 1], (uint32_t)(((g - 1) >> 1) & 1))) {
            give_up(AXB_ERR_WAIT_TMEM_FULL);
            fail = true;
          }
          tc_fence_after();
          float* red2 = red + 4 * NCOL;
#pragma unroll
          for (int c = 0; c < NCOL; ++c) {
            const float ws = warp_sum(l_thr[c]);
            if (lane == 0) red2[warp * NCOL + c] = ws;
          }
          quit = softmax_bar_or(fail || *abort_flag != 0);       // also orders the row sums above
          if (quit) break;
          uint32_t o[NPAD];
          tmem_ld_32x16(tO, o);
          if (NPAD == 32) tmem_ld_32x16(tO + 16, o + 16);
          tmem_ld_wait();
          tc_fence_before();
          mbar_arrive(&o_free[nq & 1]);         // the accumulator may be overwritten by the unit after next
#pragma unroll
          for (int c = 0; c < NCOL; ++c) {
            if (c < ncols) {
              const float l_tot = red2[c] + red2[NCOL + c] + red2[2 * NCOL + c] + red2[3 * NCOL + c];
              const long long bh = (long long)(cur.b0 + c / rep) * Hq + cur.hk * rep + c % rep;
              if (out != nullptr) {
                out[bh * PP_D + tid] = __float2bfloat16(l_tot > 0.f ? __uint_as_float(o[c]) / l_tot : 0.f);
              } else {
                const long long idx = bh * nslots + slot0 + cur.sp;
                part_o[idx * PP_D + tid] = __uint_as_float(o[c]);
                if (tid == 0) {
                  part_ml[idx * 2] = m_run[c];
                  part_ml[idx * 2 + 1] = l_tot;
                }
              }
            }
          }
          ++nq;
        }
      }
      mbar_arrive(&ring_empty[n % PP_RING]);
    }
  }

  // ---- shut down: every role has left its loop (on success all loads were consumed; after an error the producer
  // has waited for the ones in flight)
  tc_fence_before();
  __syncthreads();
  if (warp == 5) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::TCOLS);
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
  // query rows as [sequence][head][128]; one box = the rep heads of a kv head for the sequences of one item, 64 dims wide
  const int rep = Hq / Hkv;
  const int grp_seqs = 32 / rep < B ? 32 / rep : B;        // a box never exceeds the tensor
  CUtensorMap tmQ1, tmQg;
  rc = make_tmap_3d(&tmQ1, q, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, PP_D, Hq, B, PP_D * 2, q_row_stride * 2, 64, rep, 1, true);
  if (rc) return rc;
  rc = make_tmap_3d(&tmQg, q, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, PP_D, Hq, B, PP_D * 2, q_row_stride * 2, 64, rep, grp_seqs, true);
  if (rc) return rc;
  if (cudaMemsetAsync(counters, 0, 2 * sizeof(unsigned int), s) != cudaSuccess) return AXB_LAUNCH_CUDA_ERROR;
  const bool direct = n_groups == 0 && nsplit == 1;          // no prefix items, one split: the result needs no merge
  const int nslots = n_groups == 0 ? nsplit : nsplit + nsplit_p;
  float* part_o = reinterpret_cast<float*>(scratch);
  float* part_ml = part_o + (long long)B * Hq * nslots * PP_D;
  const float sl2 = softmax_scale * 1.4426950408889634f;
  // suffix items: one sequence each, slots [0, nsplit); they neutralise the prefix slots of unshared sequences
  const int total_s = B * Hkv * nsplit;
  paged_decode_persist_kernel<8><<<persist_grid(total_s), PP_THREADS, PpCfg<8>::SMEM, s>>>(
      tmK, tmV, tmQ1, 64 * 2 * rep, block_table, max_pages, seq_first, seq_one, seq_page0, seq_keys, B,
      0, nsplit, n_groups == 0 ? 0 : nsplit_p, part_o, part_ml, direct ? (__nv_bfloat16*)out : nullptr, Hq, Hkv, nsplit, nslots,
      sl2, counters, status);
  rc = check_launch();
  if (rc || direct) return rc;
  if (n_groups > 0) {
    // prefix items: one group each, slots [nsplit, nsplit + nsplit_p)
    const int total_p = n_groups * Hkv * nsplit_p;
    paged_decode_persist_kernel<32><<<persist_grid(total_p), PP_THREADS, PpCfg<32>::SMEM, s>>>(
        tmK, tmV, tmQg, 64 * 2 * rep * grp_seqs, block_table, max_pages, grp_first, grp_size, grp_zero, grp_keys,
        n_groups, nsplit, 0, 0, part_o, part_ml, nullptr, Hq, Hkv, nsplit_p, nslots, sl2, counters + 1, status);
    rc = check_launch();
    if (rc) return rc;
  }
  pp_merge_slots_kernel<<<B * Hq, PP_D, 0, s>>>(part_o, part_ml, (__nv_bfloat16*)out, nslots);
  return check_launch();
}
