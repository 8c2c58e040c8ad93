// Mixture-of-experts routing and token movement.
//
//   route     softmax over the expert logits of a token, top-k (ties broken by the lower expert id),
//             optional renormalisation of the k weights; with replay ids the selection is taken from
//             the sampler's routing (-1 entries fall back to the computed choice) while the weights
//             are always recomputed from this model's logits.
//   align     assigns every (token, slot) a row in an expert-sorted, 128-row-padded buffer. The order
//             inside an expert is token order, obtained by counting — no atomics, so the layout and
//             every sum that depends on it are reproducible.
//   gather    x_sorted[row] = x[token] (padding rows zero)
//   combine   out[token] = sum_j w[token][j] * y_sorted[row(token, j)]   — router weights applied to
//             the expert OUTPUT (after the second projection), as the sampler does
//   combine_bwd  dy_sorted[row] = w * dout[token];  dw[token][j] = <dout[token], y_sorted[row]>
#include "host_utils.h"
#include "debug.cuh"
#include "ptx.cuh"

namespace axb {

constexpr int MOE_MAX_EXPERTS = 256;
constexpr int MOE_MAX_TOPK = 16;
constexpr int MOE_PAD = 128;

// One warp per token. logits fp32 [T][E]; ids int32 [T][k]; weights fp32 [T][k]; replay int32 [T][k] or null.
__global__ void moe_route_kernel(const float* __restrict__ logits, const int* __restrict__ replay,
                                 int* __restrict__ ids, float* __restrict__ weights, long long T, int E, int k,
                                 int normalize) {
  const long long t = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (t >= T) return;
  constexpr int PER = MOE_MAX_EXPERTS / 32;
  float p[PER];
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    const int e = lane + 32 * i;
    p[i] = e < E ? logits[t * E + e] : -INFINITY;
    mx = fmaxf(mx, p[i]);
  }
  mx = warp_max(mx);
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    p[i] = (lane + 32 * i) < E ? __expf(p[i] - mx) : 0.f;
    sum += p[i];
  }
  sum = warp_sum(sum);
  const float inv = 1.f / sum;
  float prob[PER];
#pragma unroll
  for (int i = 0; i < PER; ++i) prob[i] = p[i] * inv;
  // selection: k rounds of warp arg-max over the not yet taken experts
  float sel_w = 0.f;      // lane j keeps the weight of slot j
  int sel_id = -1;
  float wsum = 0.f;
  for (int j = 0; j < k; ++j) {
    int forced = replay != nullptr ? replay[t * k + j] : -1;
    AXB_DEBUG_CHECK(forced < E, forced, E);          // a replayed expert id outside the model: ignored, recorded in debug builds
    if (forced >= E) forced = -1;
    float best = -1.f;
    int best_e = 0x7fffffff;
    if (forced < 0) {
#pragma unroll
      for (int i = 0; i < PER; ++i) {
        const int e = lane + 32 * i;
        if (e < E && p[i] >= 0.f && (prob[i] > best)) {
          best = prob[i];
          best_e = e;
        }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
        if (ob > best || (ob == best && oe < best_e)) {
          best = ob;
          best_e = oe;
        }
      }
    } else {
      best_e = forced;
      const float mine = (forced & 31) == lane ? prob[forced >> 5] : 0.f;   // prob[] index must be static:
      float v = 0.f;
#pragma unroll
      for (int i = 0; i < PER; ++i)
        if (i == (forced >> 5) && (forced & 31) == lane) v = prob[i];
      (void)mine;
      best = warp_sum(v);
    }
    // mark taken
#pragma unroll
    for (int i = 0; i < PER; ++i)
      if (lane + 32 * i == best_e) p[i] = -1.f;
    if (lane == j) {
      sel_w = best;
      sel_id = best_e;
    }
    wsum += best;
  }
  if (lane < k) {
    ids[t * k + lane] = sel_id;
    weights[t * k + lane] = normalize ? sel_w / wsum : sel_w;
  }
}

// Block e counts, in token order, the assignments to expert e. counts[e] = number of rows.
__global__ void moe_count_kernel(const int* __restrict__ ids, long long n, int* __restrict__ counts) {
  const int e = blockIdx.x;
  __shared__ int red[32];
  int c = 0;
  for (long long i = threadIdx.x; i < n; i += blockDim.x) c += ids[i] == e;
  c = static_cast<int>(warp_sum(static_cast<float>(c)));   // counts < 2^24: exact in fp32
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = c;
  __syncthreads();
  if (threadIdx.x == 0) {
    int s = 0;
    for (int w = 0; w < (blockDim.x >> 5); ++w) s += red[w];
    counts[e] = s;
  }
}

// offsets[e] = first row of expert e in the padded layout (offsets[E] = total padded rows);
// tile_expert[m] = expert of 128-row tile m (-1 for tiles past the end).
__global__ void moe_offsets_kernel(const int* __restrict__ counts, int E, int* __restrict__ offsets,
                                   int* __restrict__ tile_expert, int max_tiles) {
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    int off = 0;
    for (int e = 0; e < E; ++e) {
      offsets[e] = off;
      const int rows = (counts[e] + MOE_PAD - 1) / MOE_PAD * MOE_PAD;
      for (int m = off / MOE_PAD; m < (off + rows) / MOE_PAD && m < max_tiles; ++m) tile_expert[m] = e;
      off += rows;
    }
    offsets[E] = off;
    for (int m = off / MOE_PAD; m < max_tiles; ++m) tile_expert[m] = -1;
  }
}

// Block e walks the assignments in order and gives the c-th one row offsets[e] + c.
// row_of[i] (i = t*k + j) = destination row; token_of[row] = t (or -1 for padding rows, preset by the host).
__global__ void moe_positions_kernel(const int* __restrict__ ids, long long n, int k, const int* __restrict__ offsets,
                                     int* __restrict__ row_of, int* __restrict__ token_of) {
  const int e = blockIdx.x;
  __shared__ int warp_tot[32];
  __shared__ int base;
  if (threadIdx.x == 0) base = offsets[e];
  __syncthreads();
  const int nw = blockDim.x >> 5;
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  for (long long start = 0; start < n; start += blockDim.x) {
    const long long i = start + threadIdx.x;
    const bool hit = i < n && ids[i] == e;
    const unsigned bal = __ballot_sync(0xffffffffu, hit);
    if (lane == 0) warp_tot[w] = __popc(bal);
    __syncthreads();
    int before = 0;
    for (int q = 0; q < w; ++q) before += warp_tot[q];
    int total = 0;
    for (int q = 0; q < nw; ++q) total += warp_tot[q];
    if (hit) {
      const int r = base + before + __popc(bal & ((1u << lane) - 1u));
      row_of[i] = r;
      token_of[r] = static_cast<int>(i / k);
    }
    __syncthreads();
    if (threadIdx.x == 0) base += total;
    __syncthreads();
  }
}

// One warp per sorted row: copy H bf16 (H % 8 == 0) or zero-fill padding rows.
__global__ void moe_gather_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ token_of,
                                  __nv_bfloat16* __restrict__ xs, long long rows, int H) {
  const long long r = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (r >= rows) return;
  const int t = token_of[r];
  uint4* dst = reinterpret_cast<uint4*>(xs + r * H);
  if (t < 0) {
    for (int i = lane; i < H / 8; i += 32) dst[i] = make_uint4(0, 0, 0, 0);
  } else {
    const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<long long>(t) * H);
    for (int i = lane; i < H / 8; i += 32) dst[i] = src[i];
  }
}

__device__ __forceinline__ void unpack8f(const uint4 v, float* f) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __bfloat1622float2(h[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ uint4 pack8f(const float* f) {
  uint4 v;
  uint32_t* u = reinterpret_cast<uint32_t*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) u[i] = pack_bf16x2(f[2 * i], f[2 * i + 1]);
  return v;
}

// One warp per token: out[t] = sum_j w[t][j] * ys[row_of[t][j]] (slots in order: deterministic).
__global__ void moe_combine_kernel(const __nv_bfloat16* __restrict__ ys, const int* __restrict__ row_of,
                                   const float* __restrict__ w, __nv_bfloat16* __restrict__ out, long long T, int k,
                                   int H) {
  const long long t = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (t >= T) return;
  for (int i = lane; i < H / 8; i += 32) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int j = 0; j < k; ++j) {
      const int r = row_of[t * k + j];
      if (r < 0) continue;                      // assignment to an expert this rank does not hold
      const float wj = w[t * k + j];
      float v[8];
      unpack8f(reinterpret_cast<const uint4*>(ys + static_cast<long long>(r) * H)[i], v);
#pragma unroll
      for (int q = 0; q < 8; ++q) acc[q] += wj * v[q];
    }
    reinterpret_cast<uint4*>(out + t * H)[i] = pack8f(acc);
  }
}

// One warp per (token, slot): dys[row] = w * dout[t]; dw[t][j] = <dout[t], ys[row]>.
__global__ void moe_combine_bwd_kernel(const __nv_bfloat16* __restrict__ dout, const __nv_bfloat16* __restrict__ ys,
                                       const int* __restrict__ row_of, const float* __restrict__ w,
                                       __nv_bfloat16* __restrict__ dys, float* __restrict__ dw, long long n, int k,
                                       int H) {
  const long long i = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (i >= n) return;
  const long long t = i / k;
  const int r = row_of[i];
  const float wj = w[i];
  float dot = 0.f;
  for (int c = lane; c < H / 8; c += 32) {
    float g[8], y[8], o[8];
    unpack8f(reinterpret_cast<const uint4*>(dout + t * H)[c], g);
    unpack8f(reinterpret_cast<const uint4*>(ys + static_cast<long long>(r) * H)[c], y);
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      dot += g[q] * y[q];
      o[q] = wj * g[q];
    }
    reinterpret_cast<uint4*>(dys + static_cast<long long>(r) * H)[c] = pack8f(o);
  }
  dot = warp_sum(dot);
  if (lane == 0) dw[i] = dot;
}

// One warp per token: dx[t] = sum_j dxs[row_of[t][j]] (backward of gather).
__global__ void moe_scatter_sum_kernel(const __nv_bfloat16* __restrict__ dxs, const int* __restrict__ row_of,
                                       __nv_bfloat16* __restrict__ dx, long long T, int k, int H, int accumulate) {
  const long long t = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (t >= T) return;
  for (int i = lane; i < H / 8; i += 32) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (accumulate) unpack8f(reinterpret_cast<const uint4*>(dx + t * H)[i], acc);
    for (int j = 0; j < k; ++j) {
      float v[8];
      unpack8f(reinterpret_cast<const uint4*>(dxs + static_cast<long long>(row_of[t * k + j]) * H)[i], v);
#pragma unroll
      for (int q = 0; q < 8; ++q) acc[q] += v[q];
    }
    reinterpret_cast<uint4*>(dx + t * H)[i] = pack8f(acc);
  }
}

static inline int warp_grid(long long warps, int threads) {
  const long long b = (warps * 32 + threads - 1) / threads;
  return static_cast<int>(b < 1 ? 1 : b);
}

}  // namespace axb

using namespace axb;

extern "C" int axb_moe_route(const float* logits, const int* replay, int* ids, float* weights, long long T, int E,
                             int k, int normalize, void* stream) {
  if (T <= 0 || E <= 0 || E > MOE_MAX_EXPERTS || k <= 0 || k > MOE_MAX_TOPK || k > E) return AXB_LAUNCH_BAD_ARG;
  moe_route_kernel<<<warp_grid(T, 256), 256, 0, (cudaStream_t)stream>>>(logits, replay, ids, weights, T, E, k, normalize);
  return check_launch();
}

// ids int32 [T*k]. Outputs: counts [E], offsets [E+1], tile_expert [max_tiles], row_of [T*k], token_of
// [max_tiles*128] (filled with -1 for padding). max_tiles >= (T*k + E*127) / 128. Ids outside [0, E) (experts held by
// another rank) get no row: row_of stays -1 and the combine skips them.
extern "C" int axb_moe_align(const int* ids, long long T, int k, int E, int* counts, int* offsets, int* tile_expert,
                             int max_tiles, int* row_of, int* token_of, void* stream) {
  if (T <= 0 || E <= 0 || E > MOE_MAX_EXPERTS || k <= 0) return AXB_LAUNCH_BAD_ARG;
  if (static_cast<long long>(max_tiles) * MOE_PAD < T * k + static_cast<long long>(E) * (MOE_PAD - 1) - (MOE_PAD - 1) * 0)
    if (static_cast<long long>(max_tiles) * MOE_PAD < T * k) return AXB_LAUNCH_BAD_ARG;
  cudaStream_t s = (cudaStream_t)stream;
  if (cudaMemsetAsync(token_of, 0xff, sizeof(int) * static_cast<size_t>(max_tiles) * MOE_PAD, s) != cudaSuccess)
    return AXB_LAUNCH_CUDA_ERROR;
  if (cudaMemsetAsync(row_of, 0xff, sizeof(int) * static_cast<size_t>(T) * k, s) != cudaSuccess) return AXB_LAUNCH_CUDA_ERROR;
  moe_count_kernel<<<E, 256, 0, s>>>(ids, T * k, counts);
  moe_offsets_kernel<<<1, 32, 0, s>>>(counts, E, offsets, tile_expert, max_tiles);
  moe_positions_kernel<<<E, 256, 0, s>>>(ids, T * k, k, offsets, row_of, token_of);
  return check_launch();
}

extern "C" int axb_moe_gather(const void* x, const int* token_of, void* xs, long long rows, int H, void* stream) {
  if (rows <= 0 || H % 8 != 0) return AXB_LAUNCH_BAD_ARG;
  moe_gather_kernel<<<warp_grid(rows, 256), 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)x, token_of,
                                                                           (__nv_bfloat16*)xs, rows, H);
  return check_launch();
}

extern "C" int axb_moe_combine(const void* ys, const int* row_of, const float* w, void* out, long long T, int k, int H,
                               void* stream) {
  if (T <= 0 || H % 8 != 0) return AXB_LAUNCH_BAD_ARG;
  moe_combine_kernel<<<warp_grid(T, 256), 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)ys, row_of, w,
                                                                         (__nv_bfloat16*)out, T, k, H);
  return check_launch();
}

extern "C" int axb_moe_combine_bwd(const void* dout, const void* ys, const int* row_of, const float* w, void* dys,
                                   float* dw, long long T, int k, int H, void* stream) {
  if (T <= 0 || H % 8 != 0) return AXB_LAUNCH_BAD_ARG;
  moe_combine_bwd_kernel<<<warp_grid(T * k, 256), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)dout, (const __nv_bfloat16*)ys, row_of, w, (__nv_bfloat16*)dys, dw, T * k, k, H);
  return check_launch();
}

extern "C" int axb_moe_scatter_sum(const void* dxs, const int* row_of, void* dx, long long T, int k, int H,
                                   int accumulate, void* stream) {
  if (T <= 0 || H % 8 != 0) return AXB_LAUNCH_BAD_ARG;
  moe_scatter_sum_kernel<<<warp_grid(T, 256), 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)dxs, row_of,
                                                                             (__nv_bfloat16*)dx, T, k, H, accumulate);
  return check_launch();
}

// ------------------------------------------------------------------ expert parallelism over peer memory
// W ranks, each with its own tokens and E/W of the experts. Tokens travel to the rank that owns their
// expert and back through NVLink peer memory, written and read directly by these kernels — there is no
// all-to-all collective and no staging copy:
//   layout     from the W x E matrix of per-rank expert counts (every rank's row sits in its symmetric
//              buffer) each rank derives, identically, where its assignments land on the owners
//              (expert-major, then source rank, then token order; 128-row padded per expert) and, for
//              the experts it owns, the row offsets / tile map of its grouped GEMMs.
//   dispatch   xs_owner[row] = x[token]                     (peer store)
//   combine    out[token] = sum_j w_j * ys_owner(j)[row_j]   (peer load)
//   combine_bwd  dys_owner[row] = w * dout[token] (peer store); dw = <dout[token], ys_owner[row]> (peer load)
//   collect    dx[token] = sum_j dxs_owner(j)[row_j]         (peer load)
namespace axb {

struct EpPeers {
  void* p[8];
};

// One block. counts[s] = rank s's int32 [E] (peer pointers). Outputs (all local):
//   my_base[e]      first row, on the owner of e, of THIS rank's assignments to e
//   offsets[le]     row offsets of the local experts (le = 0..E/W), offsets[E/W] = rows in use
//   tile_expert[m]  local expert of 128-row tile m (-1 past the end)
__global__ void moe_ep_layout_kernel(EpPeers counts, int world, int rank, int E, int* __restrict__ my_base,
                                     int* __restrict__ offsets, int* __restrict__ tile_expert, int max_tiles) {
  const int epr = E / world;
  __shared__ int exp_rows[MOE_MAX_EXPERTS];     // padded rows of every expert
  __shared__ int before_me[MOE_MAX_EXPERTS];    // rows of lower-ranked sources inside the expert
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int tot = 0, pre = 0;
    for (int s = 0; s < world; ++s) {
      const int c = reinterpret_cast<const volatile int*>(counts.p[s])[e];
      if (s < rank) pre += c;
      tot += c;
    }
    exp_rows[e] = (tot + MOE_PAD - 1) / MOE_PAD * MOE_PAD;
    before_me[e] = pre;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int o = 0; o < world; ++o) {          // owner o: its experts are laid out from row 0
      int off = 0;
      for (int le = 0; le < epr; ++le) {
        const int e = o * epr + le;
        my_base[e] = off + before_me[e];
        if (o == rank) {
          offsets[le] = off;
          for (int m = off / MOE_PAD; m < (off + exp_rows[e]) / MOE_PAD && m < max_tiles; ++m) tile_expert[m] = le;
        }
        off += exp_rows[e];
      }
      if (o == rank) {
        offsets[epr] = off;
        for (int m = off / MOE_PAD; m < max_tiles; ++m) tile_expert[m] = -1;
      }
    }
  }
}

// One warp per assignment i = t*k + j.
__global__ void moe_ep_dispatch_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ ids,
                                       const int* __restrict__ row_of, EpPeers xs, long long n, int k, int H, int epr) {
  const long long i = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (i >= n) return;
  const uint4* src = reinterpret_cast<const uint4*>(x + (i / k) * H);
  uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(xs.p[ids[i] / epr]) +
                                        static_cast<long long>(row_of[i]) * H);
  for (int c = lane; c < H / 8; c += 32) dst[c] = src[c];
}

__global__ void moe_ep_combine_kernel(EpPeers ys, const int* __restrict__ ids, const int* __restrict__ row_of,
                                      const float* __restrict__ w, __nv_bfloat16* __restrict__ out, long long T, int k,
                                      int H, int epr) {
  const long long t = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (t >= T) return;
  for (int c = lane; c < H / 8; c += 32) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int j = 0; j < k; ++j) {
      const long long i = t * k + j;
      const __nv_bfloat16* base = reinterpret_cast<const __nv_bfloat16*>(ys.p[ids[i] / epr]);
      float v[8];
      unpack8f(reinterpret_cast<const uint4*>(base + static_cast<long long>(row_of[i]) * H)[c], v);
      const float wj = w[i];
#pragma unroll
      for (int q = 0; q < 8; ++q) acc[q] += wj * v[q];
    }
    reinterpret_cast<uint4*>(out + t * H)[c] = pack8f(acc);
  }
}

__global__ void moe_ep_combine_bwd_kernel(const __nv_bfloat16* __restrict__ dout, EpPeers ys, EpPeers dys,
                                          const int* __restrict__ ids, const int* __restrict__ row_of,
                                          const float* __restrict__ w, float* __restrict__ dw, long long n, int k, int H,
                                          int epr) {
  const long long i = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (i >= n) return;
  const int o = ids[i] / epr;
  const long long r = row_of[i];
  const __nv_bfloat16* y = reinterpret_cast<const __nv_bfloat16*>(ys.p[o]) + r * H;
  __nv_bfloat16* d = reinterpret_cast<__nv_bfloat16*>(dys.p[o]) + r * H;
  const float wj = w[i];
  float dot = 0.f;
  for (int c = lane; c < H / 8; c += 32) {
    float g[8], yv[8], ov[8];
    unpack8f(reinterpret_cast<const uint4*>(dout + (i / k) * H)[c], g);
    unpack8f(reinterpret_cast<const uint4*>(y)[c], yv);
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      dot += g[q] * yv[q];
      ov[q] = wj * g[q];
    }
    reinterpret_cast<uint4*>(d)[c] = pack8f(ov);
  }
  dot = warp_sum(dot);
  if (lane == 0) dw[i] = dot;
}

__global__ void moe_ep_collect_kernel(EpPeers dxs, const int* __restrict__ ids, const int* __restrict__ row_of,
                                      __nv_bfloat16* __restrict__ dx, long long T, int k, int H, int epr) {
  const long long t = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (t >= T) return;
  for (int c = lane; c < H / 8; c += 32) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int j = 0; j < k; ++j) {
      const long long i = t * k + j;
      const __nv_bfloat16* base = reinterpret_cast<const __nv_bfloat16*>(dxs.p[ids[i] / epr]);
      float v[8];
      unpack8f(reinterpret_cast<const uint4*>(base + static_cast<long long>(row_of[i]) * H)[c], v);
#pragma unroll
      for (int q = 0; q < 8; ++q) acc[q] += v[q];
    }
    reinterpret_cast<uint4*>(dx + t * H)[c] = pack8f(acc);
  }
}

static int fill_peers(EpPeers& out, const unsigned long long* ptrs, int world) {
  if (world < 1 || world > 8) return AXB_LAUNCH_BAD_ARG;
  for (int i = 0; i < 8; ++i) out.p[i] = reinterpret_cast<void*>(ptrs[i < world ? i : 0]);
  return AXB_LAUNCH_OK;
}

}  // namespace axb

// Step 1 (before the barrier): counts of this rank's assignments per expert into its symmetric slot.
extern "C" int axb_moe_ep_count(const int* ids, long long T, int k, int E, int* counts, void* stream) {
  if (T <= 0 || E <= 0 || E > MOE_MAX_EXPERTS) return AXB_LAUNCH_BAD_ARG;
  moe_count_kernel<<<E, 256, 0, (cudaStream_t)stream>>>(ids, T * k, counts);
  return check_launch();
}

// Step 2 (after the barrier): layout from all ranks' counts, then this rank's destination rows.
// scratch_token_of: int32 [>= max rows any owner can hold] (written, not used by the caller).
extern "C" int axb_moe_ep_layout(const unsigned long long* count_ptrs, int world, int rank, const int* ids, long long T,
                                 int k, int E, int* my_base, int* offsets, int* tile_expert, int max_tiles, int* row_of,
                                 int* scratch_token_of, void* stream) {
  EpPeers c;
  if (int rc = fill_peers(c, count_ptrs, world)) return rc;
  if (E % world != 0 || E > MOE_MAX_EXPERTS || T <= 0) return AXB_LAUNCH_BAD_ARG;
  cudaStream_t s = (cudaStream_t)stream;
  moe_ep_layout_kernel<<<1, 256, 0, s>>>(c, world, rank, E, my_base, offsets, tile_expert, max_tiles);
  moe_positions_kernel<<<E, 256, 0, s>>>(ids, T * k, k, my_base, row_of, scratch_token_of);
  return check_launch();
}

extern "C" int axb_moe_ep_dispatch(const void* x, const int* ids, const int* row_of, const unsigned long long* xs_ptrs,
                                   int world, long long T, int k, int H, int E, void* stream) {
  EpPeers p;
  if (int rc = fill_peers(p, xs_ptrs, world)) return rc;
  if (H % 8 != 0 || T <= 0) return AXB_LAUNCH_BAD_ARG;
  moe_ep_dispatch_kernel<<<warp_grid(T * k, 256), 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)x, ids, row_of, p,
                                                                                 T * k, k, H, E / world);
  return check_launch();
}

extern "C" int axb_moe_ep_combine(const unsigned long long* ys_ptrs, int world, const int* ids, const int* row_of,
                                  const float* w, void* out, long long T, int k, int H, int E, void* stream) {
  EpPeers p;
  if (int rc = fill_peers(p, ys_ptrs, world)) return rc;
  if (H % 8 != 0 || T <= 0) return AXB_LAUNCH_BAD_ARG;
  moe_ep_combine_kernel<<<warp_grid(T, 256), 256, 0, (cudaStream_t)stream>>>(p, ids, row_of, w, (__nv_bfloat16*)out, T, k, H,
                                                                            E / world);
  return check_launch();
}

extern "C" int axb_moe_ep_combine_bwd(const void* dout, const unsigned long long* ys_ptrs,
                                      const unsigned long long* dys_ptrs, int world, const int* ids, const int* row_of,
                                      const float* w, float* dw, long long T, int k, int H, int E, void* stream) {
  EpPeers y, d;
  if (int rc = fill_peers(y, ys_ptrs, world)) return rc;
  if (int rc = fill_peers(d, dys_ptrs, world)) return rc;
  if (H % 8 != 0 || T <= 0) return AXB_LAUNCH_BAD_ARG;
  moe_ep_combine_bwd_kernel<<<warp_grid(T * k, 256), 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)dout, y, d, ids,
                                                                                    row_of, w, dw, T * k, k, H, E / world);
  return check_launch();
}

extern "C" int axb_moe_ep_collect(const unsigned long long* dxs_ptrs, int world, const int* ids, const int* row_of,
                                  void* dx, long long T, int k, int H, int E, void* stream) {
  EpPeers p;
  if (int rc = fill_peers(p, dxs_ptrs, world)) return rc;
  if (H % 8 != 0 || T <= 0) return AXB_LAUNCH_BAD_ARG;
  moe_ep_collect_kernel<<<warp_grid(T, 256), 256, 0, (cudaStream_t)stream>>>(p, ids, row_of, (__nv_bfloat16*)dx, T, k, H,
                                                                            E / world);
  return check_launch();
}
