// Memory-bound fused kernels of the decoder layer: RMSNorm (+residual) forward/backward,
// per-head QK-RMSNorm + rotary embedding forward/backward, SwiGLU forward/backward,
// embedding gather / scatter-add. All use 16-byte vector accesses on bf16 rows; the hidden
// size must be a multiple of 8.
#include "ptx.cuh"
#include "host_utils.h"
#include "debug.cuh"

namespace axb {

__device__ __forceinline__ void unpack8(const uint4& v, float* f) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 t = __bfloat1622float2(h[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ uint4 pack8(const float* f) {
  uint4 v;
  v.x = pack_bf16x2(f[0], f[1]);
  v.y = pack_bf16x2(f[2], f[3]);
  v.z = pack_bf16x2(f[4], f[5]);
  v.w = pack_bf16x2(f[6], f[7]);
  return v;
}

template <int THREADS>
__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  __syncthreads();
  if (l == 0) red[w] = v;
  __syncthreads();
  float r = (l < THREADS / 32) ? red[l] : 0.f;
  r = warp_sum(r);
  return r;
}

// ------------------------------------------------------------------------------ RMSNorm fwd
// y = bf16(x' * rstd * w) where x' = x (+ delta). When delta != null the sum is also written
// to xsum (the new residual stream). rstd[T] is saved for the backward pass.
constexpr int NORM_THREADS = 256;
__global__ void __launch_bounds__(NORM_THREADS)
rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ delta,
                   const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ xsum,
                   __nv_bfloat16* __restrict__ y, float* __restrict__ rstd, int H, float eps) {
  __shared__ float red[NORM_THREADS / 32];
  grid_dependency_wait();     // launched as a programmatic dependent: the producer of x / delta has completed from here on
  grid_launch_dependents();   // a GEMM launched as a programmatic dependent may start streaming its weights now
  const long long row = blockIdx.x;
  const int nv = H / 8;
  const uint4* xv = reinterpret_cast<const uint4*>(x + row * H);
  const uint4* dv = delta ? reinterpret_cast<const uint4*>(delta + row * H) : nullptr;
  uint4* sv = xsum ? reinterpret_cast<uint4*>(xsum + row * H) : nullptr;
  float ss = 0.f;
  for (int i = threadIdx.x; i < nv; i += NORM_THREADS) {
    float f[8];
    unpack8(xv[i], f);
    if (dv) {
      float g[8];
      unpack8(dv[i], g);
#pragma unroll
      for (int k = 0; k < 8; ++k) f[k] += g[k];
      uint4 s = pack8(f);
      sv[i] = s;
      unpack8(s, f);  // normalise the rounded residual, as a separate add kernel would
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) ss += f[k] * f[k];
  }
  ss = block_sum<NORM_THREADS>(ss, red);
  const float r = rsqrtf(ss / H + eps);
  if (threadIdx.x == 0 && rstd) rstd[row] = r;
  const uint4* src = dv ? reinterpret_cast<const uint4*>(sv) : xv;
  const uint4* wv = reinterpret_cast<const uint4*>(w);
  uint4* yv = reinterpret_cast<uint4*>(y + row * H);
  for (int i = threadIdx.x; i < nv; i += NORM_THREADS) {
    float f[8], g[8];
    unpack8(src[i], f);
    unpack8(wv[i], g);
#pragma unroll
    for (int k = 0; k < 8; ++k) f[k] = f[k] * r * g[k];
    yv[i] = pack8(f);
  }
}

// ------------------------------------------------------------------------------ RMSNorm bwd
// dx = dres + rstd * (dy*w - xhat * mean(dy*w*xhat));  dw_partial[block] = sum_rows dy * xhat.
// Each block walks rows blockIdx.x, blockIdx.x + gridDim.x, ... and keeps its dw slice in
// registers (MAXV vectors of 8 per thread, H <= NORM_THREADS*8*MAXV).
template <int MAXV>
__global__ void __launch_bounds__(NORM_THREADS)
rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                   const __nv_bfloat16* __restrict__ w, const float* __restrict__ rstd,
                   const __nv_bfloat16* __restrict__ dres, __nv_bfloat16* __restrict__ dx,
                   float* __restrict__ dw_partial, int T, int H) {
  __shared__ float red[NORM_THREADS / 32];
  const int nv = H / 8;
  float dwacc[MAXV][8];
  float wreg[MAXV][8];
#pragma unroll
  for (int v = 0; v < MAXV; ++v) {
    const int i = threadIdx.x + v * NORM_THREADS;
#pragma unroll
    for (int k = 0; k < 8; ++k) dwacc[v][k] = 0.f;
    if (i < nv) unpack8(reinterpret_cast<const uint4*>(w)[i], wreg[v]);
  }
  for (long long row = blockIdx.x; row < T; row += gridDim.x) {
    const uint4* dyv = reinterpret_cast<const uint4*>(dy + row * H);
    const uint4* xv = reinterpret_cast<const uint4*>(x + row * H);
    const float r = rstd[row];
    float g[MAXV][8], xh[MAXV][8];
    float dot = 0.f;
#pragma unroll
    for (int v = 0; v < MAXV; ++v) {
      const int i = threadIdx.x + v * NORM_THREADS;
      if (i < nv) {
        float a[8];
        unpack8(dyv[i], a);
        unpack8(xv[i], xh[v]);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          xh[v][k] *= r;
          dwacc[v][k] += a[k] * xh[v][k];
          g[v][k] = a[k] * wreg[v][k];
          dot += g[v][k] * xh[v][k];
        }
      }
    }
    dot = block_sum<NORM_THREADS>(dot, red) / H;
    uint4* dxv = reinterpret_cast<uint4*>(dx + row * H);
    const uint4* drv = dres ? reinterpret_cast<const uint4*>(dres + row * H) : nullptr;
#pragma unroll
    for (int v = 0; v < MAXV; ++v) {
      const int i = threadIdx.x + v * NORM_THREADS;
      if (i < nv) {
        float o[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) o[k] = r * (g[v][k] - xh[v][k] * dot);
        if (drv) {
          float d[8];
          unpack8(drv[i], d);
#pragma unroll
          for (int k = 0; k < 8; ++k) o[k] += d[k];
        }
        dxv[i] = pack8(o);
      }
    }
  }
#pragma unroll
  for (int v = 0; v < MAXV; ++v) {
    const int i = threadIdx.x + v * NORM_THREADS;
    if (i < nv) {
      float* o = dw_partial + (long long)blockIdx.x * H + i * 8;
#pragma unroll
      for (int k = 0; k < 8; ++k) o[k] = dwacc[v][k];
    }
  }
}

// out[c] (+)= sum_p partial[p][c]   (deterministic column reduction of the dw partials)
__global__ void reduce_partials_kernel(const float* __restrict__ partial, float* __restrict__ out,
                                       int P, int H, int accumulate) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= H) return;
  float s = 0.f;
  for (int p = 0; p < P; ++p) s += partial[(long long)p * H + c];
  out[c] = accumulate ? out[c] + s : s;
}

// ------------------------------------------------------------------------------ QK-norm + RoPE
// One warp per (token, head). Head dim D = 128 (4 elements per lane) or 64 (2 per lane, EPL).
// Rotary pairs element i with i + D/2 (rotate-half convention); lanes l and l^16 are partners.
// Heads [0,Hq) are queries, [Hq,Hq+Hkv) keys (both optionally RMS-normalised with their own
// weight, then rotated), [Hq+Hkv, Hq+2Hkv) values (copied).
// Optional second destination of the K / V rows: the paged KV cache ([num_pages][Hkv][page][D]).
struct QkvCacheDst {
  __nv_bfloat16* kcache;
  __nv_bfloat16* vcache;
  const int* tok_seq;        // block-table row of every token
  const int* block_table;
  int max_pages, num_pages, page;
};

template <int EPL>
__global__ void __launch_bounds__(256)
qknorm_rope_fwd_kernel(const __nv_bfloat16* __restrict__ qkv, __nv_bfloat16* __restrict__ out,
                       const __nv_bfloat16* __restrict__ qw, const __nv_bfloat16* __restrict__ kw,
                       const int* __restrict__ pos, const float* __restrict__ cos_t,
                       const float* __restrict__ sin_t, long long n_items, int Hq, int Hkv,
                       float eps, QkvCacheDst cache) {
  constexpr int D = EPL * 32;
  grid_dependency_wait();
  grid_launch_dependents();
  const int lane = threadIdx.x & 31;
  const int HT = Hq + 2 * Hkv;
  for (long long item = (long long)blockIdx.x * 8 + (threadIdx.x >> 5); item < n_items;
       item += (long long)gridDim.x * 8) {
    const long long t = item / HT;
    const int h = (int)(item - t * HT);
    const __nv_bfloat16* src = qkv + item * D + lane * EPL;
    __nv_bfloat16* dst = out + item * D + lane * EPL;
    float f[EPL];
    if (EPL == 4) {
      uint2 v = *reinterpret_cast<const uint2*>(src);
      float2 a = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&v.x));
      float2 b = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&v.y));
      f[0] = a.x; f[1] = a.y; f[EPL - 2] = b.x; f[EPL - 1] = b.y;
    } else {
      float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(src));
      f[0] = a.x; f[1] = a.y;
    }
    if (h < Hq + Hkv) {
      const __nv_bfloat16* nw = h < Hq ? qw : kw;
      if (nw != nullptr) {
        float ss = 0.f;
#pragma unroll
        for (int k = 0; k < EPL; ++k) ss += f[k] * f[k];
        ss = warp_sum(ss);
        const float r = rsqrtf(ss / D + eps);
#pragma unroll
        for (int k = 0; k < EPL; ++k) f[k] = f[k] * r * __bfloat162float(nw[lane * EPL + k]);
      }
      const int p = pos[t];
      const int fi = (lane & 15) * EPL;
      const float* cp = cos_t + (long long)p * (D / 2) + fi;
      const float* sp = sin_t + (long long)p * (D / 2) + fi;
#pragma unroll
      for (int k = 0; k < EPL; ++k) {
        const float other = __shfl_xor_sync(0xffffffffu, f[k], 16);
        const float c = cp[k], s = sp[k];
        f[k] = lane < 16 ? f[k] * c - other * s : f[k] * c + other * s;
      }
    }
    // sampler paths: the rotated K row and the V row also go straight to their page of the KV cache
    __nv_bfloat16* cdst = nullptr;
    if (cache.kcache != nullptr && h >= Hq) {
      const int seq = cache.tok_seq[t], p = pos[t];
      if (seq >= 0 && p >= 0) {
        const int page = cache.block_table[(long long)seq * cache.max_pages + p / cache.page];
        if (page >= 0 && page < cache.num_pages) {
          const int is_v = h >= Hq + Hkv;
          const int hk = h - Hq - is_v * Hkv;
          cdst = (is_v ? cache.vcache : cache.kcache) + (((long long)page * Hkv + hk) * cache.page + (p % cache.page)) * D + lane * EPL;
        }
      }
    }
    if (EPL == 4) {
      uint2 o;
      o.x = pack_bf16x2(f[0], f[1]);
      o.y = pack_bf16x2(f[EPL - 2], f[EPL - 1]);
      *reinterpret_cast<uint2*>(dst) = o;
      if (cdst != nullptr) *reinterpret_cast<uint2*>(cdst) = o;
    } else {
      const uint32_t o = pack_bf16x2(f[0], f[1]);
      *reinterpret_cast<uint32_t*>(dst) = o;
      if (cdst != nullptr) *reinterpret_cast<uint32_t*>(cdst) = o;
    }
  }
}

// Backward of the above: dqkv = d(raw qkv) from dout (grad of rotated/normalised output) and
// the saved raw qkv. Norm-weight grads go to per-block partials [gridDim][2][D].
template <int EPL>
__global__ void __launch_bounds__(256)
qknorm_rope_bwd_kernel(const __nv_bfloat16* __restrict__ dout, const __nv_bfloat16* __restrict__ qkv,
                       __nv_bfloat16* __restrict__ dqkv, const __nv_bfloat16* __restrict__ qw,
                       const __nv_bfloat16* __restrict__ kw, const int* __restrict__ pos,
                       const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                       float* __restrict__ dw_partial, long long n_items, int Hq, int Hkv,
                       float eps) {
  constexpr int D = EPL * 32;
  __shared__ float sdw[8][2][D];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int HT = Hq + 2 * Hkv;
  float dwq[EPL], dwk[EPL];
#pragma unroll
  for (int k = 0; k < EPL; ++k) dwq[k] = dwk[k] = 0.f;
  for (long long item = (long long)blockIdx.x * 8 + warp; item < n_items;
       item += (long long)gridDim.x * 8) {
    const long long t = item / HT;
    const int h = (int)(item - t * HT);
    float g[EPL], x[EPL];
#pragma unroll
    for (int k = 0; k < EPL; ++k) {
      g[k] = __bfloat162float(dout[item * D + lane * EPL + k]);
      x[k] = __bfloat162float(qkv[item * D + lane * EPL + k]);
    }
    if (h < Hq + Hkv) {
      const int p = pos[t];
      const int fi = (lane & 15) * EPL;
      const float* cp = cos_t + (long long)p * (D / 2) + fi;
      const float* sp = sin_t + (long long)p * (D / 2) + fi;
#pragma unroll
      for (int k = 0; k < EPL; ++k) {
        const float other = __shfl_xor_sync(0xffffffffu, g[k], 16);
        const float c = cp[k], s = sp[k];
        g[k] = lane < 16 ? g[k] * c + other * s : g[k] * c - other * s;
      }
      const __nv_bfloat16* nw = h < Hq ? qw : kw;
      if (nw != nullptr) {
        float ss = 0.f;
#pragma unroll
        for (int k = 0; k < EPL; ++k) ss += x[k] * x[k];
        ss = warp_sum(ss);
        const float r = rsqrtf(ss / D + eps);
        float dot = 0.f;
        float gw[EPL];
#pragma unroll
        for (int k = 0; k < EPL; ++k) {
          const float xh = x[k] * r;
          if (h < Hq) dwq[k] += g[k] * xh; else dwk[k] += g[k] * xh;
          gw[k] = g[k] * __bfloat162float(nw[lane * EPL + k]);
          dot += gw[k] * xh;
          x[k] = xh;
        }
        dot = warp_sum(dot) / D;
#pragma unroll
        for (int k = 0; k < EPL; ++k) g[k] = r * (gw[k] - x[k] * dot);
      }
    }
#pragma unroll
    for (int k = 0; k < EPL; ++k) dqkv[item * D + lane * EPL + k] = __float2bfloat16(g[k]);
  }
  if (dw_partial != nullptr) {
#pragma unroll
    for (int k = 0; k < EPL; ++k) {
      sdw[warp][0][lane * EPL + k] = dwq[k];
      sdw[warp][1][lane * EPL + k] = dwk[k];
    }
    __syncthreads();
    for (int i = threadIdx.x; i < 2 * D; i += 256) {
      float s = 0.f;
      for (int w8 = 0; w8 < 8; ++w8) s += sdw[w8][i / D][i % D];
      dw_partial[(long long)blockIdx.x * 2 * D + i] = s;
    }
  }
}

// ------------------------------------------------------------------------------ SwiGLU
// gu is [T][2F] (gate | up); a[T][F] = silu(gate) * up.
__global__ void swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ a,
                                  long long T, int F) {
  grid_dependency_wait();
  grid_launch_dependents();   // see rmsnorm_fwd_kernel
  const int fv = F / 8;
  const long long n = T * fv;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / fv;
    const int c = (int)(i - t * fv);
    float g[8], u[8];
    unpack8(reinterpret_cast<const uint4*>(gu + t * 2 * F)[c], g);
    unpack8(reinterpret_cast<const uint4*>(gu + t * 2 * F + F)[c], u);
#pragma unroll
    for (int k = 0; k < 8; ++k) g[k] = g[k] / (1.f + __expf(-g[k])) * u[k];
    reinterpret_cast<uint4*>(a + t * F)[c] = pack8(g);
  }
}
__global__ void swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ da, const __nv_bfloat16* __restrict__ gu,
                                  __nv_bfloat16* __restrict__ dgu, long long T, int F) {
  const int fv = F / 8;
  const long long n = T * fv;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / fv;
    const int c = (int)(i - t * fv);
    float g[8], u[8], d[8];
    unpack8(reinterpret_cast<const uint4*>(gu + t * 2 * F)[c], g);
    unpack8(reinterpret_cast<const uint4*>(gu + t * 2 * F + F)[c], u);
    unpack8(reinterpret_cast<const uint4*>(da + t * F)[c], d);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float s = 1.f / (1.f + __expf(-g[k]));
      const float silu = g[k] * s;
      const float dg = d[k] * u[k] * (s + silu * (1.f - s));
      u[k] = d[k] * silu;
      g[k] = dg;
    }
    reinterpret_cast<uint4*>(dgu + t * 2 * F)[c] = pack8(g);
    reinterpret_cast<uint4*>(dgu + t * 2 * F + F)[c] = pack8(u);
  }
}

// ------------------------------------------------------------------------------ embedding
__global__ void embedding_fwd_kernel(const int* __restrict__ ids, const __nv_bfloat16* __restrict__ table,
                                     __nv_bfloat16* __restrict__ out, long long T, int H, int V) {
  const int nv = H / 8;
  for (long long t = blockIdx.x; t < T; t += gridDim.x) {
    int id = ids[t];
    AXB_DEBUG_CHECK(id >= 0 && id < V, id, V);
    id = id < 0 ? 0 : (id >= V ? V - 1 : id);
    const uint4* src = reinterpret_cast<const uint4*>(table + (long long)id * H);
    uint4* dst = reinterpret_cast<uint4*>(out + t * H);
    for (int i = threadIdx.x; i < nv; i += blockDim.x) dst[i] = src[i];
  }
}
// dtable[ids[t]] += dy[t]  (fp32 atomics)
__global__ void embedding_bwd_kernel(const int* __restrict__ ids, const __nv_bfloat16* __restrict__ dy,
                                     float* __restrict__ dtable, long long T, int H, int V) {
  for (long long t = blockIdx.x; t < T; t += gridDim.x) {
    const int id = ids[t];
    AXB_DEBUG_CHECK(id >= 0 && id < V, id, V);
    if (id < 0 || id >= V) continue;
    for (int i = threadIdx.x; i < H; i += blockDim.x)
      atomicAdd(dtable + (long long)id * H + i, __bfloat162float(dy[t * H + i]));
  }
}

// y = a + b (bf16), used for residual adds that are not fused into a norm.
__global__ void add_bf16_kernel(const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ b,
                                __nv_bfloat16* __restrict__ y, long long n8) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n8;
       i += (long long)gridDim.x * blockDim.x) {
    float f[8], g[8];
    unpack8(reinterpret_cast<const uint4*>(a)[i], f);
    unpack8(reinterpret_cast<const uint4*>(b)[i], g);
#pragma unroll
    for (int k = 0; k < 8; ++k) f[k] += g[k];
    reinterpret_cast<uint4*>(y)[i] = pack8(f);
  }
}

}  // namespace axb

using namespace axb;

static inline int grid_for(long long n, int threads, int per_sm = 8) {
  long long b = (n + threads - 1) / threads;
  long long cap = (long long)sm_count() * per_sm;
  return (int)(b < 1 ? 1 : (b > cap ? cap : b));
}

extern "C" int axb_rmsnorm_fwd(const void* x, const void* delta, const void* w, void* xsum, void* y,
                               float* rstd, long long T, int H, float eps, void* stream) {
  if (H % 8 != 0 || T <= 0) return AXB_LAUNCH_BAD_ARG;
  if (delta != nullptr && xsum == nullptr) return AXB_LAUNCH_BAD_ARG;
  const int rc = launch_dependent(rmsnorm_fwd_kernel, dim3((unsigned)T), dim3(NORM_THREADS), 0, (cudaStream_t)stream,
                                  (const __nv_bfloat16*)x, (const __nv_bfloat16*)delta, (const __nv_bfloat16*)w,
                                  (__nv_bfloat16*)xsum, (__nv_bfloat16*)y, rstd, H, eps);
  return rc ? rc : check_launch();
}

// Number of row-partials rmsnorm_bwd writes; scratch must hold that many rows of H floats.
extern "C" int axb_rmsnorm_bwd_partials(long long T) {
  long long cap = (long long)sm_count() * 4;
  return (int)(T < cap ? T : cap);
}

extern "C" int axb_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd,
                               const void* dres, void* dx, float* dw, int dw_accumulate,
                               float* scratch, long long T, int H, void* stream) {
  if (H % 8 != 0 || T <= 0 || H > NORM_THREADS * 8 * 4) return AXB_LAUNCH_BAD_ARG;
  const int P = axb_rmsnorm_bwd_partials(T);
  cudaStream_t s = (cudaStream_t)stream;
  const int nv = H / 8;
#define AXB_NB(MAXV)                                                                       \
  rmsnorm_bwd_kernel<MAXV><<<P, NORM_THREADS, 0, s>>>(                                     \
      (const __nv_bfloat16*)dy, (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, rstd,    \
      (const __nv_bfloat16*)dres, (__nv_bfloat16*)dx, scratch, (int)T, H)
  if (nv <= NORM_THREADS) AXB_NB(1);
  else if (nv <= 2 * NORM_THREADS) AXB_NB(2);
  else AXB_NB(4);
#undef AXB_NB
  int rc = check_launch();
  if (rc) return rc;
  reduce_partials_kernel<<<(H + 255) / 256, 256, 0, s>>>(scratch, dw, P, H, dw_accumulate);
  return check_launch();
}

static int launch_qknorm_rope_fwd(const void* qkv, void* out, const void* qw, const void* kw, const int* pos,
                                  const float* cos_t, const float* sin_t, long long T, int Hq, int Hkv, int D,
                                  float eps, QkvCacheDst cache, void* stream) {
  if ((D != 128 && D != 64) || T <= 0) return AXB_LAUNCH_BAD_ARG;
  const long long n = T * (Hq + 2 * Hkv);
  const int grid = grid_for(n, 8, 16);
  int rc;
  if (D == 128)
    rc = launch_dependent(qknorm_rope_fwd_kernel<4>, dim3(grid), dim3(256), 0, (cudaStream_t)stream, (const __nv_bfloat16*)qkv,
                          (__nv_bfloat16*)out, (const __nv_bfloat16*)qw, (const __nv_bfloat16*)kw, pos, cos_t, sin_t, n, Hq, Hkv, eps, cache);
  else
    rc = launch_dependent(qknorm_rope_fwd_kernel<2>, dim3(grid), dim3(256), 0, (cudaStream_t)stream, (const __nv_bfloat16*)qkv,
                          (__nv_bfloat16*)out, (const __nv_bfloat16*)qw, (const __nv_bfloat16*)kw, pos, cos_t, sin_t, n, Hq, Hkv, eps, cache);
  return rc ? rc : check_launch();
}

extern "C" int axb_qknorm_rope_fwd(const void* qkv, void* out, const void* qw, const void* kw,
                                   const int* pos, const float* cos_t, const float* sin_t,
                                   long long T, int Hq, int Hkv, int D, float eps, void* stream) {
  return launch_qknorm_rope_fwd(qkv, out, qw, kw, pos, cos_t, sin_t, T, Hq, Hkv, D, eps, QkvCacheDst{}, stream);
}

// Same, and the rotated K rows / the V rows of token t are also written to page
// block_table[tok_seq[t]][pos[t] / page] of the KV cache (one launch instead of two on the sampler paths).
extern "C" int axb_qknorm_rope_fwd_kv(const void* qkv, void* out, const void* qw, const void* kw, const int* pos,
                                      const float* cos_t, const float* sin_t, long long T, int Hq, int Hkv, int D,
                                      float eps, void* kcache, void* vcache, const int* tok_seq,
                                      const int* block_table, int max_pages, int num_pages, int page, void* stream) {
  if (kcache == nullptr || vcache == nullptr || tok_seq == nullptr || block_table == nullptr || page <= 0) return AXB_LAUNCH_BAD_ARG;
  QkvCacheDst c{(__nv_bfloat16*)kcache, (__nv_bfloat16*)vcache, tok_seq, block_table, max_pages, num_pages, page};
  return launch_qknorm_rope_fwd(qkv, out, qw, kw, pos, cos_t, sin_t, T, Hq, Hkv, D, eps, c, stream);
}

extern "C" int axb_qknorm_rope_bwd_partials(long long T, int Hq, int Hkv) {
  return grid_for(T * (Hq + 2 * Hkv), 8, 4);
}

// dqw/dkw: fp32 [D] each, may be null when the model has no QK-norm. scratch: partials*2*D floats.
extern "C" int axb_qknorm_rope_bwd(const void* dout, const void* qkv, void* dqkv, const void* qw,
                                   const void* kw, const int* pos, const float* cos_t,
                                   const float* sin_t, float* dqw, float* dkw, int dw_accumulate,
                                   float* scratch, long long T, int Hq, int Hkv, int D, float eps,
                                   void* stream) {
  if ((D != 128 && D != 64) || T <= 0) return AXB_LAUNCH_BAD_ARG;
  const long long n = T * (Hq + 2 * Hkv);
  const int grid = axb_qknorm_rope_bwd_partials(T, Hq, Hkv);
  cudaStream_t s = (cudaStream_t)stream;
  float* part = qw != nullptr ? scratch : nullptr;
  if (D == 128)
    qknorm_rope_bwd_kernel<4><<<grid, 256, 0, s>>>(
        (const __nv_bfloat16*)dout, (const __nv_bfloat16*)qkv, (__nv_bfloat16*)dqkv,
        (const __nv_bfloat16*)qw, (const __nv_bfloat16*)kw, pos, cos_t, sin_t, part, n, Hq, Hkv, eps);
  else
    qknorm_rope_bwd_kernel<2><<<grid, 256, 0, s>>>(
        (const __nv_bfloat16*)dout, (const __nv_bfloat16*)qkv, (__nv_bfloat16*)dqkv,
        (const __nv_bfloat16*)qw, (const __nv_bfloat16*)kw, pos, cos_t, sin_t, part, n, Hq, Hkv, eps);
  int rc = check_launch();
  if (rc || part == nullptr) return rc;
  // partial layout [grid][2][D] -> columns 0..D-1 are dqw, D..2D-1 are dkw
  reduce_partials_kernel<<<(2 * D + 255) / 256, 256, 0, s>>>(scratch, scratch + (long long)grid * 2 * D,
                                                            grid, 2 * D, 0);
  rc = check_launch();
  if (rc) return rc;
  // second tiny pass: move (or add) the 2*D sums into dqw / dkw
  reduce_partials_kernel<<<1, 256, 0, s>>>(scratch + (long long)grid * 2 * D, dqw, 1, D, dw_accumulate);
  reduce_partials_kernel<<<1, 256, 0, s>>>(scratch + (long long)grid * 2 * D + D, dkw, 1, D, dw_accumulate);
  return check_launch();
}

extern "C" int axb_swiglu_fwd(const void* gu, void* a, long long T, int F, void* stream) {
  if (F % 8 != 0 || T <= 0) return AXB_LAUNCH_BAD_ARG;
  const int rc = launch_dependent(swiglu_fwd_kernel, dim3(grid_for(T * (F / 8), 256)), dim3(256), 0, (cudaStream_t)stream,
                                  (const __nv_bfloat16*)gu, (__nv_bfloat16*)a, T, F);
  return rc ? rc : check_launch();
}
extern "C" int axb_swiglu_bwd(const void* da, const void* gu, void* dgu, long long T, int F, void* stream) {
  if (F % 8 != 0 || T <= 0) return AXB_LAUNCH_BAD_ARG;
  swiglu_bwd_kernel<<<grid_for(T * (F / 8), 256), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)da, (const __nv_bfloat16*)gu, (__nv_bfloat16*)dgu, T, F);
  return check_launch();
}
extern "C" int axb_embedding_fwd(const int* ids, const void* table, void* out, long long T, int H, int V,
                                 void* stream) {
  if (H % 8 != 0 || T <= 0) return AXB_LAUNCH_BAD_ARG;
  embedding_fwd_kernel<<<grid_for(T, 1, 16), 128, 0, (cudaStream_t)stream>>>(
      ids, (const __nv_bfloat16*)table, (__nv_bfloat16*)out, T, H, V);
  return check_launch();
}
extern "C" int axb_embedding_bwd(const int* ids, const void* dy, float* dtable, long long T, int H, int V,
                                 void* stream) {
  if (T <= 0) return AXB_LAUNCH_BAD_ARG;
  embedding_bwd_kernel<<<grid_for(T, 1, 16), 256, 0, (cudaStream_t)stream>>>(
      ids, (const __nv_bfloat16*)dy, dtable, T, H, V);
  return check_launch();
}
extern "C" int axb_add_bf16(const void* a, const void* b, void* y, long long n, void* stream) {
  if (n % 8 != 0 || n <= 0) return AXB_LAUNCH_BAD_ARG;
  add_bf16_kernel<<<grid_for(n / 8, 256), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)a, (const __nv_bfloat16*)b, (__nv_bfloat16*)y, n / 8);
  return check_launch();
}

// --------------------------------------------------------- RMSNorm backward, workspace built in
#include "rmsnorm_bwd_static.h"
#include <cstdio>

static __device__ __align__(256) float g_rmsnorm_bwd_scratch[AXB_RMSNORM_BWD_STATIC_MAX_FLOATS];

namespace {
constexpr int kMaxDevices = 64;
float* g_scratch_ptr[kMaxDevices] = {};
thread_local char g_static_err[192] = "";

int static_scratch(float** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    snprintf(g_static_err, sizeof(g_static_err), "rmsnorm_bwd_static: no usable current device (%s)",
             cudaGetErrorString(e));
    return AXB_LAUNCH_CUDA_ERROR;
  }
  if (g_scratch_ptr[dev] == nullptr) {
    float* p = nullptr;
    e = cudaGetSymbolAddress((void**)&p, g_rmsnorm_bwd_scratch);
    if (e != cudaSuccess || p == nullptr) {
      snprintf(g_static_err, sizeof(g_static_err),
               "rmsnorm_bwd_static: cudaGetSymbolAddress failed on device %d (%s)", dev,
               cudaGetErrorString(e));
      return AXB_LAUNCH_CUDA_ERROR;
    }
    g_scratch_ptr[dev] = p;
  }
  *out = g_scratch_ptr[dev];
  return AXB_LAUNCH_OK;
}
}  // namespace

extern "C" const char* axb_rmsnorm_bwd_static_error(void) { return g_static_err; }

extern "C" int axb_rmsnorm_bwd_static_setup(void) {
  float* p = nullptr;
  g_static_err[0] = 0;
  return static_scratch(&p);
}

extern "C" int axb_rmsnorm_bwd_static(const void* dy, const void* x, const void* w, const float* rstd,
                                      const void* dres, void* dx, float* dw, int dw_accumulate,
                                      long long T, int H, void* stream) {
  g_static_err[0] = 0;
  if (H % 8 != 0 || H <= 0 || T <= 0 || H > NORM_THREADS * 8 * 4) {
    snprintf(g_static_err, sizeof(g_static_err),
             "rmsnorm_bwd_static: need T > 0 and H a multiple of 8 up to %d (got T=%lld H=%d)",
             NORM_THREADS * 8 * 4, T, H);
    return AXB_LAUNCH_BAD_ARG;
  }
  const long long need = (long long)axb_rmsnorm_bwd_partials(T) * H;
  if (need > (long long)AXB_RMSNORM_BWD_STATIC_MAX_FLOATS) {
    snprintf(g_static_err, sizeof(g_static_err),
             "rmsnorm_bwd_static: T=%lld H=%d needs %lld workspace floats, the built-in workspace "
             "holds %d; use axb_rmsnorm_bwd with a caller-owned workspace",
             T, H, need, AXB_RMSNORM_BWD_STATIC_MAX_FLOATS);
    return AXB_LAUNCH_TOO_LARGE;
  }
  // The workspace address is looked up for the CURRENT device; a stream that lives on another device
  // would run the kernel there with this device's address, so such a call is refused.
  if (stream != nullptr) {
    int cur = -1, sdev = -1;
    if (cudaGetDevice(&cur) == cudaSuccess && cudaStreamGetDevice((cudaStream_t)stream, &sdev) == cudaSuccess &&
        sdev != cur) {
      snprintf(g_static_err, sizeof(g_static_err),
               "rmsnorm_bwd_static: the stream belongs to device %d but device %d is current", sdev, cur);
      return AXB_LAUNCH_BAD_ARG;
    }
  }
  float* scratch = nullptr;
  int rc = static_scratch(&scratch);
  if (rc) return rc;
  rc = axb_rmsnorm_bwd(dy, x, w, rstd, dres, dx, dw, dw_accumulate, scratch, T, H, stream);
  if (rc)
    snprintf(g_static_err, sizeof(g_static_err), "rmsnorm_bwd_static: launch failed with code %d", rc);
  return rc;
}
