// Kernels that move data between GPUs through NVLink peer memory (plain peer loads / stores on
// pointers obtained from symmetric-memory or CUDA-IPC mappings; no NCCL, no TMA multicast).
//
//   peer_barrier        device-side barrier over per-rank signal pads, bounded wait + status word
//   zero1_reduce        gradient reduce-scatter: sum this rank's shard over all ranks' fp32 grad
//                       buffers (peer loads), emit the reduced shard and sum-of-squares partials
//   zero1_adamw_bcast   sharded AdamW on the reduced shard (clip coefficient / skip flag read on the
//                       device) + all-gather fused as peer STORES of the new bf16 values into every
//                       rank's parameter buffer
//   peer_allreduce      one-launch all-reduce of a small bf16 vector (push to every rank's staging slot,
//                       per-block flags, fixed-order sum); epoch kept on the device, graph-replayable
//   p2p_copy_plan       trainer -> sampler weight sync: executes a compiled RoutingTable plan (strided
//                       2-D slice copies between arbitrary ranks) in ONE launch; optional fused
//                       bf16 -> fp8(e4m3) 128x128 block-scaled quantisation on the way
//
// Every wait on another rank is bounded (AXB_PEER_WAIT_CYCLES) and reports AXB_ERR_WAIT_PEER in the
// status word instead of spinning forever.
#include "ptx.cuh"
#include "host_utils.h"
#include "debug.cuh"
#include <cuda_fp8.h>

namespace axb {

#ifndef AXB_PEER_WAIT_CYCLES
#define AXB_PEER_WAIT_CYCLES (1ll << 32)   // ~2 s
#endif

constexpr int MAX_RANKS = 16;

struct PeerPtrs {
  void* p[MAX_RANKS];
};

__device__ __forceinline__ void st_release_sys(unsigned int* addr, unsigned int v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int* addr) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
  return v;
}

// Each rank owns a pad of `world` 32-bit slots. Arriving at the barrier with epoch e means writing e
// into slot[rank] of every peer's pad, then waiting until every slot of the own pad holds >= e.
// One block, >= world threads. Epochs must increase by one per barrier on every rank.
__global__ void peer_barrier_kernel(PeerPtrs pads, int rank, int world, unsigned int epoch, int* status) {
  const int t = threadIdx.x;
  __threadfence_system();
  if (t < world) {
    st_release_sys(reinterpret_cast<unsigned int*>(pads.p[t]) + rank, epoch);
    const unsigned int* mine = reinterpret_cast<const unsigned int*>(pads.p[rank]) + t;
    const long long t0 = clock64();
    while (static_cast<int>(ld_acquire_sys(mine) - epoch) < 0) {
      if (clock64() - t0 > AXB_PEER_WAIT_CYCLES) {
        report_error(status, AXB_ERR_WAIT_PEER);
        break;
      }
      __nanosleep(200);
    }
  }
  __syncthreads();
  __threadfence_system();
}

// out[i] = sum_r grads[r][lo + i] for i in [0, n); partial[block] = sum of out^2 over the block's slice.
// The own rank is read first so local traffic overlaps the remote request latency.
__global__ void __launch_bounds__(256)
zero1_reduce_kernel(PeerPtrs grads, int rank, int world, long long lo, long long n, float* __restrict__ out,
                    float* __restrict__ partial) {
  __shared__ float red[8];
  float ss = 0.f;
  const long long n4 = n / 4;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4;
       i += (long long)gridDim.x * blockDim.x) {
    float4 acc = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(grads.p[rank]) + lo)[i];
#pragma unroll 1
    for (int k = 1; k < world; ++k) {
      const int r = (rank + k) % world;
      const float4 v = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(grads.p[r]) + lo)[i];
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    reinterpret_cast<float4*>(out)[i] = acc;
    ss += acc.x * acc.x + acc.y * acc.y + acc.z * acc.z + acc.w * acc.w;
  }
  for (long long i = n4 * 4 + (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    float acc = 0.f;
    for (int k = 0; k < world; ++k) acc += reinterpret_cast<const float*>(grads.p[(rank + k) % world])[lo + i];
    out[i] = acc;
    ss += acc * acc;
  }
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x < 32) {
    float r = threadIdx.x < 8 ? red[threadIdx.x] : 0.f;
    r = warp_sum(r);
    if (threadIdx.x == 0) partial[blockIdx.x] = r;
  }
}

// AdamW on the reduced shard; the new bf16 value of element lo + i is stored into EVERY rank's
// parameter buffer (the all-gather). state: [sumsq, norm, clip coef, skip flag] as in optim.cu.
__global__ void __launch_bounds__(256)
zero1_adamw_bcast_kernel(float* __restrict__ master, const float* __restrict__ grad, float* __restrict__ m,
                         float* __restrict__ v, PeerPtrs params, int world, long long lo, long long n, float lr,
                         float beta1, float beta2, float eps, float wd, float bc1, float bc2,
                         const float* __restrict__ state) {
  if (state != nullptr && state[3] != 0.f) return;
  const float coef = state != nullptr ? state[2] : 1.f;
  const float inv_bc1 = 1.f / bc1, inv_sqrt_bc2 = rsqrtf(bc2);
  const long long n8 = n / 8;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n8;
       i += (long long)gridDim.x * blockDim.x) {
    // 8 consecutive elements per thread as two 16-byte vectors per array (the shard arrays start on
    // allocation boundaries): scalar loads at a 32-byte stride would use an eighth of every sector
    float p[8];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const float4 g4 = reinterpret_cast<const float4*>(grad)[i * 2 + h];
      float4 m4 = reinterpret_cast<const float4*>(m)[i * 2 + h];
      float4 v4 = reinterpret_cast<const float4*>(v)[i * 2 + h];
      float4 w4 = reinterpret_cast<const float4*>(master)[i * 2 + h];
      auto upd = [&](float g, float& mi, float& vi, float& w) {
        g *= coef;
        mi = beta1 * mi + (1.f - beta1) * g;
        vi = beta2 * vi + (1.f - beta2) * g * g;
        w -= lr * wd * w;
        w -= lr * (mi * inv_bc1) / (sqrtf(vi) * inv_sqrt_bc2 + eps);
      };
      upd(g4.x, m4.x, v4.x, w4.x);
      upd(g4.y, m4.y, v4.y, w4.y);
      upd(g4.z, m4.z, v4.z, w4.z);
      upd(g4.w, m4.w, v4.w, w4.w);
      reinterpret_cast<float4*>(m)[i * 2 + h] = m4;
      reinterpret_cast<float4*>(v)[i * 2 + h] = v4;
      reinterpret_cast<float4*>(master)[i * 2 + h] = w4;
      p[4 * h + 0] = w4.x;
      p[4 * h + 1] = w4.y;
      p[4 * h + 2] = w4.z;
      p[4 * h + 3] = w4.w;
    }
    uint4 o;
    o.x = pack_bf16x2(p[0], p[1]);
    o.y = pack_bf16x2(p[2], p[3]);
    o.z = pack_bf16x2(p[4], p[5]);
    o.w = pack_bf16x2(p[6], p[7]);
#pragma unroll 1
    for (int r = 0; r < world; ++r)
      reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(params.p[r]) + lo)[i] = o;
  }
  for (long long j = n8 * 8 + (long long)blockIdx.x * blockDim.x + threadIdx.x; j < n;
       j += (long long)gridDim.x * blockDim.x) {
    const float g = grad[j] * coef;
    const float mi = beta1 * m[j] + (1.f - beta1) * g;
    const float vi = beta2 * v[j] + (1.f - beta2) * g * g;
    m[j] = mi;
    v[j] = vi;
    float w = master[j];
    w -= lr * wd * w;
    w -= lr * (mi * inv_bc1) / (sqrtf(vi) * inv_sqrt_bc2 + eps);
    master[j] = w;
    for (int r = 0; r < world; ++r) reinterpret_cast<__nv_bfloat16*>(params.p[r])[lo + j] = __float2bfloat16(w);
  }
}

// ------------------------------------------------------------------------------ weight-sync plan
// One descriptor = one strided 2-D slice copy src[rows][cols] -> dst[rows][cols] (element offsets and
// row strides in elements of the bf16 source / destination buffers). quant: 0 = bf16 copy,
// 1 = quantise to fp8 e4m3 with one fp32 scale per 128x128 block (dst buffers are then fp8 bytes and
// dst_scale_off indexes the fp32 scale buffer of the destination rank, row-major over blocks).
struct CopyDesc {
  long long src_off, dst_off;
  int rows, cols;
  long long src_stride, dst_stride;
  int dst_rank, quant;
  long long dst_scale_off;
  int scale_cols, pad;
};

__global__ void __launch_bounds__(256)
p2p_copy_plan_kernel(const __nv_bfloat16* __restrict__ src, PeerPtrs dst, PeerPtrs dst_scales,
                     const CopyDesc* __restrict__ descs, const long long* __restrict__ work_prefix, int n_desc,
                     long long total_work) {
  // Work items: 16-byte vectors (bf16 copy) laid out descriptor after descriptor; work_prefix[d] is
  // the first item of descriptor d. Each block claims a contiguous span so its stores stay sequential.
  __shared__ int s_desc;
  const long long per_block = (total_work + gridDim.x - 1) / gridDim.x;
  const long long w0 = (long long)blockIdx.x * per_block;
  const long long w1 = min(total_work, w0 + per_block);
  if (w0 >= w1) return;
  if (threadIdx.x == 0) {
    int lo = 0, hi = n_desc - 1;            // last descriptor whose prefix <= w0
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if (work_prefix[mid] <= w0) lo = mid; else hi = mid - 1;
    }
    s_desc = lo;
  }
  __syncthreads();
  int d = s_desc;
  for (long long w = w0 + threadIdx.x; w < w1; w += blockDim.x) {
    while (d + 1 < n_desc && work_prefix[d + 1] <= w) ++d;
    const CopyDesc& c = descs[d];
    AXB_DEBUG_CHECK(c.dst_rank >= 0 && c.dst_rank < MAX_RANKS && dst.p[c.dst_rank] != nullptr, c.dst_rank, d);
    if (c.dst_rank < 0 || c.dst_rank >= MAX_RANKS || dst.p[c.dst_rank] == nullptr) continue;
    const long long local = w - work_prefix[d];
    const int vec_per_row = (c.cols + 7) / 8;
    const int r = (int)(local / vec_per_row);
    const int cv = (int)(local - (long long)r * vec_per_row);
    const __nv_bfloat16* s = src + c.src_off + (long long)r * c.src_stride + cv * 8;
    __nv_bfloat16* t = reinterpret_cast<__nv_bfloat16*>(dst.p[c.dst_rank]) + c.dst_off + (long long)r * c.dst_stride + cv * 8;
    const int left = c.cols - cv * 8;
    if (left >= 8 && ((reinterpret_cast<uintptr_t>(s) | reinterpret_cast<uintptr_t>(t)) & 15) == 0) {
      *reinterpret_cast<uint4*>(t) = *reinterpret_cast<const uint4*>(s);
    } else {
      for (int k = 0; k < left && k < 8; ++k) t[k] = s[k];
    }
  }
}

// Quantising variant: one CTA per 128x128 block of a descriptor. amax over the block, scale =
// amax / 448 (1 when amax is 0 or not finite), fp8 = sat(x / scale); the scale is what the consumer
// multiplies by (the "weight_scale_inv" of block-scaled fp8 checkpoints).
struct QuantTile {
  int desc, block_row, block_col, pad;
};
// One 128 x 128 (or ragged edge) tile: bf16 -> e4m3 with one scale = amax / 448, by 256 threads.
// Full tiles whose rows are 16-byte aligned on both sides stay in registers between the maximum and the cast:
// thread t holds 8 vectors of 8 elements (rows t / 16 + 16 k), reads each once and stores 8-byte vectors.
__device__ __forceinline__ void quant_tile_128(const __nv_bfloat16* __restrict__ src, long long src_stride,
                                               unsigned char* __restrict__ dst, long long dst_stride, int nr, int nc,
                                               float* red, float* s_scale, float* scale_out) {
  const bool fast = nr == 128 && nc == 128 && (src_stride & 7) == 0 && (dst_stride & 7) == 0 &&
                    (reinterpret_cast<uintptr_t>(src) & 15) == 0 && (reinterpret_cast<uintptr_t>(dst) & 7) == 0;
  uint4 v[8];
  float amax = 0.f;
  if (fast) {
    const int r = threadIdx.x >> 4, cv = (threadIdx.x & 15) * 8;
#pragma unroll
    for (int k = 0; k < 8; ++k) v[k] = *reinterpret_cast<const uint4*>(src + (long long)(r + 16 * k) * src_stride + cv);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v[k]);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(h[j]);
        amax = fmaxf(amax, fmaxf(fabsf(f.x), fabsf(f.y)));
      }
    }
  } else {
    for (int i = threadIdx.x; i < nr * 128; i += blockDim.x) {
      const int r = i >> 7, cc = i & 127;
      if (cc < nc) amax = fmaxf(amax, fabsf(__bfloat162float(src[(long long)r * src_stride + cc])));
    }
  }
  amax = warp_max(amax);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
  __syncthreads();
  if (threadIdx.x == 0) {
    float a = red[0];
    for (int w = 1; w < 8; ++w) a = fmaxf(a, red[w]);
    const float scale = (a > 0.f && isfinite(a)) ? a / 448.f : 1.f;
    *s_scale = scale;
    *scale_out = scale;
  }
  __syncthreads();
  const float inv = 1.f / *s_scale;
  if (fast) {
    const int r = threadIdx.x >> 4, cv = (threadIdx.x & 15) * 8;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v[k]);
      uint32_t w[2];
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const float2 f0 = __bfloat1622float2(h[2 * j]), f1 = __bfloat1622float2(h[2 * j + 1]);
        const __nv_fp8x4_e4m3 q(make_float4(f0.x * inv, f0.y * inv, f1.x * inv, f1.y * inv));
        w[j] = *reinterpret_cast<const uint32_t*>(&q);
      }
      *reinterpret_cast<uint2*>(dst + (long long)(r + 16 * k) * dst_stride + cv) = make_uint2(w[0], w[1]);
    }
  } else {
    for (int i = threadIdx.x; i < nr * 128; i += blockDim.x) {
      const int r = i >> 7, cc = i & 127;
      if (cc < nc) {
        const __nv_fp8_e4m3 f(__bfloat162float(src[(long long)r * src_stride + cc]) * inv);
        dst[(long long)r * dst_stride + cc] = *reinterpret_cast<const unsigned char*>(&f);
      }
    }
  }
  __syncthreads();      // red / s_scale are reused by the caller's next tile
}

__global__ void __launch_bounds__(256)
p2p_quant_plan_kernel(const __nv_bfloat16* __restrict__ src, PeerPtrs dst, PeerPtrs dst_scales,
                      const CopyDesc* __restrict__ descs, const QuantTile* __restrict__ tiles, int n_tiles) {
  __shared__ float red[8];
  __shared__ float s_scale;
  for (int ti = blockIdx.x; ti < n_tiles; ti += gridDim.x) {
    const QuantTile q = tiles[ti];
    const CopyDesc& c = descs[q.desc];
    const int r0 = q.block_row * 128, c0 = q.block_col * 128;
    const int nr = min(128, c.rows - r0), nc = min(128, c.cols - c0);
    quant_tile_128(src + c.src_off + (long long)r0 * c.src_stride + c0, c.src_stride,
                   reinterpret_cast<unsigned char*>(dst.p[c.dst_rank]) + c.dst_off + (long long)r0 * c.dst_stride + c0, c.dst_stride,
                   nr, nc, red, &s_scale,
                   reinterpret_cast<float*>(dst_scales.p[c.dst_rank]) + c.dst_scale_off + (long long)q.block_row * c.scale_cols + q.block_col);
  }
}

// Stand-alone bf16 -> fp8 e4m3 128x128 block quantisation of a local [rows][cols] matrix.
__global__ void __launch_bounds__(256)
fp8_block_quant_kernel(const __nv_bfloat16* __restrict__ x, unsigned char* __restrict__ y, float* __restrict__ scales,
                       int rows, int cols, long long ldx, long long ldy) {
  __shared__ float red[8];
  __shared__ float s_scale;
  const int bc = (cols + 127) / 128;
  const int r0 = blockIdx.y * 128, c0 = blockIdx.x * 128;
  quant_tile_128(x + (long long)r0 * ldx + c0, ldx, y + (long long)r0 * ldy + c0, ldy, min(128, rows - r0), min(128, cols - c0), red,
                 &s_scale, scales + (long long)blockIdx.y * bc + blockIdx.x);
}

// One-launch all-reduce of a small bf16 vector (a decode step's activations under tensor parallelism).
// Every rank owns, in symmetric memory, staging [2 turns][world slots][cap] bf16 and flags
// [2][world][max_blocks] u32. Block b of rank r handles elements [b * chunk, (b + 1) * chunk):
//   1. stores its chunk of x into slot r of EVERY rank's staging (peer stores over NVLink),
//   2. fences, then sets flag (turn, r, b) on every rank to the call's epoch,
//   3. waits (bounded) until its own flags (turn, 0..world-1, b) reached the epoch,
//   4. sums the world slots of its own staging in rank order (every rank gets the same bits) into out.
// The epoch lives in device memory (state[0], bumped by the block that finishes last), so the launch has
// no per-call arguments and can be replayed from a CUDA graph. turn = epoch & 1: a rank that runs one
// call ahead writes the other half, and it cannot run two ahead because step 3 of the call in between
// needs this rank's flags. out may alias x. No block waits for another block of the same launch.
__global__ void __launch_bounds__(256)
peer_allreduce_kernel(PeerPtrs bufs, int rank, int world, const __nv_bfloat16* x, __nv_bfloat16* out, long long n,
                      long long chunk, long long cap, long long flag_off_bytes, int max_blocks, unsigned int* state,
                      int* status) {
  __shared__ unsigned int s_epoch;
  const int tid = threadIdx.x;
  if (tid == 0) s_epoch = *reinterpret_cast<volatile unsigned int*>(state) + 1u;
  __syncthreads();
  const unsigned int e = s_epoch;
  const int turn = static_cast<int>(e & 1u);
  const long long lo = blockIdx.x * chunk, hi = min(n, lo + chunk);
  for (int d = 1; d <= world; ++d) {
    const int p = (rank + d) % world;
    __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(bufs.p[p]) + (static_cast<long long>(turn) * world + rank) * cap;
    for (long long i = lo + tid * 8; i < hi; i += 256 * 8)
      *reinterpret_cast<uint4*>(dst + i) = *reinterpret_cast<const uint4*>(x + i);
  }
  __threadfence_system();
  __syncthreads();
  if (tid < world) {
    unsigned int* theirs = reinterpret_cast<unsigned int*>(reinterpret_cast<char*>(bufs.p[tid]) + flag_off_bytes) +
                           (static_cast<long long>(turn) * world + rank) * max_blocks + blockIdx.x;
    st_release_sys(theirs, e);
    const unsigned int* mine = reinterpret_cast<const unsigned int*>(reinterpret_cast<const char*>(bufs.p[rank]) + flag_off_bytes) +
                               (static_cast<long long>(turn) * world + tid) * max_blocks + blockIdx.x;
    const long long t0 = clock64();
    while (static_cast<int>(ld_acquire_sys(mine) - e) < 0) {
      if (clock64() - t0 > AXB_PEER_WAIT_CYCLES) {
        report_error(status, AXB_ERR_WAIT_PEER);
        break;
      }
      __nanosleep(100);
    }
  }
  __syncthreads();
  const __nv_bfloat16* base = reinterpret_cast<const __nv_bfloat16*>(bufs.p[rank]) + static_cast<long long>(turn) * world * cap;
  for (long long i = lo + tid * 8; i < hi; i += 256 * 8) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int r = 0; r < world; ++r) {
      const uint4 v = __ldcg(reinterpret_cast<const uint4*>(base + r * cap + i));      // L2 is where the peers' stores land
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float2 f = __bfloat1622float2(h[q]);
        acc[2 * q] += f.x;
        acc[2 * q + 1] += f.y;
      }
    }
    uint4 o;
    uint32_t* u = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
    for (int q = 0; q < 4; ++q) u[q] = pack_bf16x2(acc[2 * q], acc[2 * q + 1]);
    *reinterpret_cast<uint4*>(out + i) = o;
  }
  __syncthreads();
  if (tid == 0) {
    __threadfence();
    if (atomicAdd(state + 1, 1u) == gridDim.x - 1) {       // last block out: publish the epoch for the next launch
      state[1] = 0u;
      __threadfence();
      *reinterpret_cast<volatile unsigned int*>(state) = e;
    }
  }
}

}  // namespace axb

using namespace axb;

static int fill_ptrs(PeerPtrs& out, const unsigned long long* ptrs, int world) {
  if (world < 1 || world > MAX_RANKS) return AXB_LAUNCH_BAD_ARG;
  for (int i = 0; i < MAX_RANKS; ++i) out.p[i] = i < world ? reinterpret_cast<void*>(ptrs[i]) : nullptr;
  return AXB_LAUNCH_OK;
}

extern "C" int axb_peer_barrier(const unsigned long long* pad_ptrs, int rank, int world, unsigned int epoch,
                                int* status, void* stream) {
  PeerPtrs pads;
  if (int rc = fill_ptrs(pads, pad_ptrs, world)) return rc;
  peer_barrier_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(pads, rank, world, epoch, status);
  return check_launch();
}

// bufs: base of every rank's symmetric allocation ([2][world][cap] bf16 staging, flags at flag_off_bytes:
// [2][world][max_blocks] u32, zero before the first call). state: 2 zero-initialised u32 of this rank.
// n (a multiple of 8, <= cap) bf16 elements of x are summed over the ranks into out (may alias x).
extern "C" int axb_peer_allreduce(const unsigned long long* buf_ptrs, int rank, int world, const void* x, void* out,
                                  long long n, long long cap, long long flag_off_bytes, int max_blocks,
                                  unsigned int* state, int* status, void* stream) {
  PeerPtrs b;
  if (int rc = fill_ptrs(b, buf_ptrs, world)) return rc;
  if (n <= 0 || (n & 7) || n > cap || (cap & 7) || max_blocks < 1 || rank < 0 || rank >= world || (flag_off_bytes & 3) ||
      (reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(out) & 15))
    return AXB_LAUNCH_BAD_ARG;
  long long blocks = (n + 2047) / 2048;
  if (blocks > max_blocks) blocks = max_blocks;
  const long long chunk = ((n + blocks - 1) / blocks + 7) & ~7ll;
  blocks = (n + chunk - 1) / chunk;
  peer_allreduce_kernel<<<static_cast<int>(blocks), 256, 0, (cudaStream_t)stream>>>(
      b, rank, world, static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(out), n, chunk, cap, flag_off_bytes,
      max_blocks, state, status);
  return check_launch();
}

extern "C" int axb_zero1_partials(void) { return sm_count() * 4; }

// out: fp32 [n] reduced shard; partial: fp32 [axb_zero1_partials()].
extern "C" int axb_zero1_reduce(const unsigned long long* grad_ptrs, int rank, int world, long long lo, long long n,
                                float* out, float* partial, void* stream) {
  PeerPtrs g;
  if (int rc = fill_ptrs(g, grad_ptrs, world)) return rc;
  if (n <= 0 || (lo & 3) != 0) return AXB_LAUNCH_BAD_ARG;
  zero1_reduce_kernel<<<axb_zero1_partials(), 256, 0, (cudaStream_t)stream>>>(g, rank, world, lo, n, out, partial);
  return check_launch();
}

// state[0] = sum over ranks of stats_r[r] (rank r's sum-of-squares partial, read from rank r's own
// buffer with plain peer loads, in rank order so every rank derives the same total).
__global__ void zero1_total_kernel(PeerPtrs stats, int world, float* __restrict__ state) {
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    float t = 0.f;
    for (int r = 0; r < world; ++r) t += reinterpret_cast<const volatile float*>(stats.p[r])[r];
    state[0] = t;
  }
}

extern "C" int axb_zero1_total(const unsigned long long* stats_ptrs, int world, float* state, void* stream) {
  PeerPtrs s;
  if (int rc = fill_ptrs(s, stats_ptrs, world)) return rc;
  zero1_total_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(s, world, state);
  return check_launch();
}

extern "C" int axb_zero1_adamw_bcast(float* master, const float* grad, float* m, float* v,
                                     const unsigned long long* param_ptrs, int world, long long lo, long long n,
                                     float lr, float beta1, float beta2, float eps, float wd, float bc1, float bc2,
                                     const float* state, void* stream) {
  PeerPtrs p;
  if (int rc = fill_ptrs(p, param_ptrs, world)) return rc;
  if (n <= 0 || (lo & 7) != 0) return AXB_LAUNCH_BAD_ARG;
  if ((reinterpret_cast<uintptr_t>(master) | reinterpret_cast<uintptr_t>(grad) | reinterpret_cast<uintptr_t>(m) |
       reinterpret_cast<uintptr_t>(v)) & 15)
    return AXB_LAUNCH_BAD_ARG;      // the kernel moves 16-byte vectors
  zero1_adamw_bcast_kernel<<<sm_count() * 4, 256, 0, (cudaStream_t)stream>>>(master, grad, m, v, p, world, lo, n, lr,
                                                                            beta1, beta2, eps, wd, bc1, bc2, state);
  return check_launch();
}

// descs / work_prefix / tiles live on the device. total_work = number of 16-byte vectors (copy mode).
extern "C" int axb_p2p_copy_plan(const void* src, const unsigned long long* dst_ptrs, int world, const void* descs,
                                 const long long* work_prefix, int n_desc, long long total_work, void* stream) {
  PeerPtrs d, s;
  if (int rc = fill_ptrs(d, dst_ptrs, world)) return rc;
  fill_ptrs(s, dst_ptrs, world);
  if (n_desc <= 0 || total_work <= 0) return AXB_LAUNCH_BAD_ARG;
  long long blocks = (total_work + 2047) / 2048;
  const long long cap = (long long)sm_count() * 8;
  if (blocks > cap) blocks = cap;
  p2p_copy_plan_kernel<<<(int)blocks, 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)src, d, s, (const CopyDesc*)descs, work_prefix, n_desc, total_work);
  return check_launch();
}

extern "C" int axb_p2p_quant_plan(const void* src, const unsigned long long* dst_ptrs,
                                  const unsigned long long* scale_ptrs, int world, const void* descs,
                                  const void* tiles, int n_tiles, void* stream) {
  PeerPtrs d, s;
  if (int rc = fill_ptrs(d, dst_ptrs, world)) return rc;
  if (int rc = fill_ptrs(s, scale_ptrs, world)) return rc;
  if (n_tiles <= 0) return AXB_LAUNCH_BAD_ARG;
  int blocks = n_tiles < sm_count() * 8 ? n_tiles : sm_count() * 8;
  p2p_quant_plan_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)src, d, s,
                                                                 (const CopyDesc*)descs, (const QuantTile*)tiles, n_tiles);
  return check_launch();
}

extern "C" int axb_fp8_block_quant(const void* x, void* y, float* scales, int rows, int cols, long long ldx,
                                   long long ldy, void* stream) {
  if (rows <= 0 || cols <= 0) return AXB_LAUNCH_BAD_ARG;
  dim3 grid((cols + 127) / 128, (rows + 127) / 128);
  fp8_block_quant_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)x, (unsigned char*)y, scales,
                                                                rows, cols, ldx, ldy);
  return check_launch();
}
