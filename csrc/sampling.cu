// Token sampling with log-prob capture for the in-house sampler.
//
// One CTA per sequence row of fp32 logits [B][V]:
//   z = logits / temperature  ->  optional top-k (count radix-select on sortable float keys)
//   -> optional top-p (mass radix-select over the kept set) -> renormalise -> inverse-CDF sample
//   -> logprob of the chosen token. Two conventions, chosen per launch:
//     processed (default): under the PROCESSED distribution (after temperature / top-k / top-p,
//       renormalised over the kept set), as the reference's vLLM fork reports it
//       (install/vllm/axon.patch:635-680);
//     full vocabulary: temperature-scaled log-softmax over ALL tokens, the quantity the trainer's
//       old_log_probs hold; with top-k / top-p active this is the one importance-sampling
//       corrections should be fed, since the truncated mass only shapes the draw.
// temperature == 0 selects arg-max and reports the unscaled log-softmax of that token.
#include "ptx.cuh"
#include "host_utils.h"

namespace axb {

constexpr int SMP_THREADS = 1024;

__device__ __forceinline__ uint32_t f2key(float f) {
  const uint32_t b = __float_as_uint(f);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

__device__ __forceinline__ float block_reduce_max(float v, float* red) {
  v = warp_max(v);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float r = red[threadIdx.x & 31];
  r = warp_max(r);
  return r;
}
__device__ __forceinline__ float block_reduce_sum(float v, float* red) {
  v = warp_sum(v);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float r = red[threadIdx.x & 31];
  r = warp_sum(r);
  return r;
}

__device__ __forceinline__ uint32_t mix32(uint32_t x) {
  x ^= x >> 16; x *= 0x7feb352dU; x ^= x >> 15; x *= 0x846ca68bU; x ^= x >> 16;
  return x;
}
// Uniform in (0,1) from (seed, stream id, counter).
__device__ __forceinline__ float uniform01(unsigned long long seed, uint32_t row, uint32_t ctr) {
  uint32_t h = mix32((uint32_t)seed ^ 0x9E3779B9u);
  h = mix32(h ^ (uint32_t)(seed >> 32));
  h = mix32(h ^ (row * 0x85EBCA6Bu + 0x27d4eb2fu));
  h = mix32(h ^ (ctr * 0xC2B2AE35u + 0x165667b1u));
  return ((h >> 8) + 0.5f) * (1.0f / 16777216.0f);
}

// Radix select from the top over keys >= floor_key. by_mass = false: find the largest key K with
// count(key >= K) >= target. by_mass = true: find the largest key K with mass(key >= K) >= target.
__device__ uint32_t radix_select(const float* __restrict__ row, int V, float inv_t, float m, bool by_mass,
                                 float target, uint32_t floor_key, float* hist, uint32_t* sh_prefix,
                                 float* sh_target) {
  uint32_t prefix = 0;
  if (threadIdx.x == 0) {
    *sh_target = target;
  }
  for (int round = 0; round < 4; ++round) {
    const int shift = 24 - 8 * round;
    for (int i = threadIdx.x; i < 256; i += blockDim.x) hist[i] = 0.f;
    __syncthreads();
    const uint32_t hi_mask = round == 0 ? 0u : (0xFFFFFFFFu << (shift + 8));
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
      const float z = row[i] * inv_t;
      const uint32_t k = f2key(z);
      if (k < floor_key) continue;
      if ((k & hi_mask) != (prefix & hi_mask)) continue;
      atomicAdd(&hist[(k >> shift) & 255], by_mass ? __expf(z - m) : 1.f);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      float need = *sh_target, cum = 0.f;
      int bin = 0;
      for (int bq = 255; bq >= 0; --bq) {
        if (cum + hist[bq] >= need) {
          bin = bq;
          break;
        }
        cum += hist[bq];
        bin = bq;  // falls through to the lowest bin when the mass never reaches the target
      }
      *sh_target = need - cum;
      *sh_prefix = prefix | ((uint32_t)bin << shift);
    }
    __syncthreads();
    prefix = *sh_prefix;
  }
  return prefix;
}

__global__ void __launch_bounds__(SMP_THREADS)
sample_kernel(const float* __restrict__ logits, long long ldl, int V, const float* __restrict__ temperature,
              const int* __restrict__ top_k, const float* __restrict__ top_p, unsigned long long seed,
              const int* __restrict__ counters, int* __restrict__ tokens, float* __restrict__ logprobs,
              int full_vocab_logprob) {
  __shared__ float red[32];
  __shared__ float hist[256];
  __shared__ float seg[SMP_THREADS];
  __shared__ uint32_t sh_prefix;
  __shared__ float sh_target;
  __shared__ int sh_choice;
  const int b = blockIdx.x;
  const float* row = logits + (long long)b * ldl;
  const float temp = temperature ? temperature[b] : 1.f;
  const bool greedy = temp <= 0.f;
  const float inv_t = greedy ? 1.f : 1.f / temp;

  float mx = -INFINITY;
  int amax = 0;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    const float z = row[i] * inv_t;
    if (z > mx) {
      mx = z;
      amax = i;
    }
  }
  const float m = block_reduce_max(mx, red);

  if (greedy) {
    // smallest index among the maxima
    int cand = (mx == m) ? amax : V;
    for (int o = 16; o > 0; o >>= 1) cand = min(cand, __shfl_xor_sync(0xffffffffu, cand, o));
    __shared__ int ired[32];
    if ((threadIdx.x & 31) == 0) ired[threadIdx.x >> 5] = cand;
    __syncthreads();
    int c2 = ired[threadIdx.x & 31];
    for (int o = 16; o > 0; o >>= 1) c2 = min(c2, __shfl_xor_sync(0xffffffffu, c2, o));
    float s = 0.f;
    for (int i = threadIdx.x; i < V; i += blockDim.x) s += __expf(row[i] - m);
    s = block_reduce_sum(s, red);
    if (threadIdx.x == 0) {
      tokens[b] = c2;
      logprobs[b] = row[c2] - m - logf(s);
    }
    return;
  }

  uint32_t thr_key = 0;  // keep elements with key >= thr_key
  const int k = top_k ? top_k[b] : 0;
  if (k > 0 && k < V) thr_key = radix_select(row, V, inv_t, m, false, (float)k, 0u, hist, &sh_prefix, &sh_target);
  const float p = top_p ? top_p[b] : 1.f;
  if (p < 1.f) {
    float zk = 0.f;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
      const float z = row[i] * inv_t;
      if (f2key(z) >= thr_key) zk += __expf(z - m);
    }
    zk = block_reduce_sum(zk, red);
    const uint32_t pk = radix_select(row, V, inv_t, m, true, p * zk, thr_key, hist, &sh_prefix, &sh_target);
    thr_key = max(thr_key, pk);
  }

  // Inverse CDF over the kept set. Any fixed order of the kept elements samples the same distribution; the
  // order used is (thread, then index): thread t owns elements t, t + 1024, t + 2048, ..., so that every pass
  // over the logits is coalesced (a contiguous segment per thread would touch 32 cache lines per warp load).
  float ssum = 0.f;
  for (int i = threadIdx.x; i < V; i += SMP_THREADS) {
    const float z = row[i] * inv_t;
    if (f2key(z) >= thr_key) ssum += __expf(z - m);
  }
  seg[threadIdx.x] = ssum;
  const float total = block_reduce_sum(ssum, red);  // includes the barriers that publish seg[]
  float norm = total;                               // denominator of the reported log-prob
  if (full_vocab_logprob && thr_key != 0u) {
    float fs = 0.f;
    for (int i = threadIdx.x; i < V; i += SMP_THREADS) fs += __expf(row[i] * inv_t - m);
    norm = block_reduce_sum(fs, red);
  }
  if (threadIdx.x == 0) {
    // with per-row counters (request id and token index folded in by the caller) the draw does not depend on the row a
    // sequence happens to occupy in the batch
    const float u = uniform01(seed, counters ? 0u : (uint32_t)b, counters ? (uint32_t)counters[b] : 0u);
    float target = u * total, cum = 0.f;
    int t = 0, last_ne = 0;
    bool found = false;
    for (; t < SMP_THREADS; ++t) {
      if (seg[t] > 0.f) last_ne = t;
      if (cum + seg[t] > target) {
        found = true;
        break;
      }
      cum += seg[t];
    }
    if (!found) {            // rounding pushed the target to the very end: the last thread that kept anything
      t = last_ne;
      cum -= seg[t];
    }
    // walk the chosen thread's elements
    int choice = -1, last_kept = -1;
    for (int i = t; i < V; i += SMP_THREADS) {
      const float z = row[i] * inv_t;
      if (f2key(z) < thr_key) continue;
      last_kept = i;
      cum += __expf(z - m);
      if (cum > target) {
        choice = i;
        break;
      }
    }
    if (choice < 0) choice = last_kept >= 0 ? last_kept : 0;
    sh_choice = choice;
    tokens[b] = choice;
    logprobs[b] = row[choice] * inv_t - m - logf(norm);
  }
}

// Repetition penalty on logits of tokens already seen (HF / vLLM convention: divide positive
// logits by the penalty, multiply negative ones). seen: uint8 [B][V] presence mask.
__global__ void repetition_penalty_kernel(float* __restrict__ logits, long long ldl, int V,
                                          const unsigned char* __restrict__ seen, const float* __restrict__ penalty) {
  const int b = blockIdx.y;
  const float pen = penalty[b];
  if (pen == 1.f) return;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < V; i += gridDim.x * blockDim.x) {
    if (seen[(long long)b * V + i]) {
      float* x = logits + (long long)b * ldl + i;
      *x = *x > 0.f ? *x / pen : *x * pen;
    }
  }
}

}  // namespace axb

using namespace axb;

// temperature/top_k/top_p: per-row device arrays (null = 1.0 / off / 1.0). counters: per-row int
// mixed into the RNG stream (e.g. the decode step), may be null.
// full_vocab_logprob: 0 = log-prob under the processed (truncated, renormalised) distribution, 1 = under the
// temperature-scaled softmax over the whole vocabulary.
extern "C" int axb_sample_ex(const float* logits, long long ldl, int B, int V, const float* temperature,
                             const int* top_k, const float* top_p, unsigned long long seed, const int* counters,
                             int* tokens, float* logprobs, int full_vocab_logprob, void* stream) {
  if (B <= 0 || V <= 0) return AXB_LAUNCH_BAD_ARG;
  sample_kernel<<<B, SMP_THREADS, 0, (cudaStream_t)stream>>>(logits, ldl, V, temperature, top_k, top_p, seed,
                                                            counters, tokens, logprobs, full_vocab_logprob);
  return check_launch();
}

extern "C" int axb_sample(const float* logits, long long ldl, int B, int V, const float* temperature,
                          const int* top_k, const float* top_p, unsigned long long seed, const int* counters,
                          int* tokens, float* logprobs, void* stream) {
  return axb_sample_ex(logits, ldl, B, V, temperature, top_k, top_p, seed, counters, tokens, logprobs, 0, stream);
}

extern "C" int axb_repetition_penalty(float* logits, long long ldl, int B, int V, const unsigned char* seen,
                                      const float* penalty, void* stream) {
  if (B <= 0 || V <= 0) return AXB_LAUNCH_BAD_ARG;
  repetition_penalty_kernel<<<dim3(32, B), 256, 0, (cudaStream_t)stream>>>(logits, ldl, V, seen, penalty);
  return check_launch();
}
