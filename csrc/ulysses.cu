// Sequence <-> head exchange of Ulysses sequence parallelism as two peer-store kernels.
//
// Between the projections and the attention kernel every rank trades "all heads of my T/W tokens"
// for "my H/W heads of all T tokens" (and back after attention). The reference runs a list-based
// torch.distributed.all_to_all on q, k and v plus one on the output (axon/utils/ulysses.py:133-192),
// four collectives per attention layer with pack / unpack copies around each. Here the exchange is
// one kernel per direction: each CTA reads rows of the local activation once and stores the column
// slices straight into the symmetric buffers of the ranks that need them (NVLink peer stores, 16 bytes
// per thread), already in the layout the attention kernel consumes - q, k and v travel together.
// A device barrier (bounded) after the kernel publishes the stores.
//
//   scatter_cols:  dst_p[rank * rows + t, seg.dst + c]      = src[t, seg.src + p * seg.w + c]
//                  (tokens stay, heads are dealt out:  local [T/W, all heads] -> peers' [T, my heads])
//   scatter_rows:  dst_p[t, seg.dst + rank * seg.w + c]     = src[p * rows + t, seg.src + c]
//                  (heads stay, tokens are dealt out:  local [T, my heads]  -> peers' [T/W, all heads])
// for every destination rank p, row t < rows and up to three column segments (q | k | v).
#include "ptx.cuh"
#include "host_utils.h"

namespace axb {

constexpr int UL_MAX_RANKS = 8;
struct UlSeg {
  int src, w, dst;   // element offsets / per-rank width (multiples of 8)
};
struct UlParams {
  __nv_bfloat16* dst[UL_MAX_RANKS];
  UlSeg seg[3];
  int nseg, world, rank, rows;
  long long ld_src, ld_dst;
};

template <bool ROWS>
__global__ void __launch_bounds__(256) ulysses_scatter_kernel(const __nv_bfloat16* __restrict__ src, const UlParams p) {
  // one (destination, row) pair per blockIdx.x; threads stride over the 16-byte units of the segments
  const int per_row_units = (p.seg[0].w + (p.nseg > 1 ? p.seg[1].w : 0) + (p.nseg > 2 ? p.seg[2].w : 0)) / 8;
  for (long long item = blockIdx.x; item < static_cast<long long>(p.world) * p.rows; item += gridDim.x) {
    const int d = static_cast<int>(item / p.rows);
    const int t = static_cast<int>(item % p.rows);
    const __nv_bfloat16* srow = src + (ROWS ? (static_cast<long long>(d) * p.rows + t) : static_cast<long long>(t)) * p.ld_src;
    __nv_bfloat16* drow = p.dst[d] + (ROWS ? static_cast<long long>(t) : (static_cast<long long>(p.rank) * p.rows + t)) * p.ld_dst;
    for (int u = threadIdx.x; u < per_row_units; u += blockDim.x) {
      int c = u * 8, s = 0;
      while (s + 1 < p.nseg && c >= p.seg[s].w) {
        c -= p.seg[s].w;
        ++s;
      }
      const UlSeg sg = p.seg[s];
      const int so = ROWS ? sg.src + c : sg.src + d * sg.w + c;
      const int dof = ROWS ? sg.dst + p.rank * sg.w + c : sg.dst + c;
      *reinterpret_cast<uint4*>(drow + dof) = *reinterpret_cast<const uint4*>(srow + so);
    }
  }
}

}  // namespace axb

// segs: nseg x (src offset, per-rank width, dst offset) in elements. by_rows = 0: scatter_cols, 1: scatter_rows.
extern "C" int axb_ulysses_scatter(const void* src, long long ld_src, const unsigned long long* dst_ptrs, long long ld_dst,
                                   int world, int rank, int rows, const int* segs, int nseg, int by_rows, void* stream) {
  using namespace axb;
  if (world < 1 || world > UL_MAX_RANKS || nseg < 1 || nseg > 3 || rows <= 0 || (ld_src & 7) || (ld_dst & 7)) return AXB_LAUNCH_BAD_ARG;
  UlParams p;
  for (int i = 0; i < world; ++i) p.dst[i] = reinterpret_cast<__nv_bfloat16*>(dst_ptrs[i]);
  for (int i = 0; i < nseg; ++i) {
    p.seg[i] = UlSeg{segs[3 * i], segs[3 * i + 1], segs[3 * i + 2]};
    if ((p.seg[i].src & 7) || (p.seg[i].w & 7) || (p.seg[i].dst & 7) || p.seg[i].w <= 0) return AXB_LAUNCH_BAD_ARG;
  }
  p.nseg = nseg;
  p.world = world;
  p.rank = rank;
  p.rows = rows;
  p.ld_src = ld_src;
  p.ld_dst = ld_dst;
  const long long items = static_cast<long long>(world) * rows;
  const int grid = static_cast<int>(items < 148 * 16 ? items : 148 * 16);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (by_rows) ulysses_scatter_kernel<true><<<grid, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(src), p);
  else ulysses_scatter_kernel<false><<<grid, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(src), p);
  return check_launch();
}
