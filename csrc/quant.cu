// Weight quantisers used when synced weights are handed to a low-precision sampler:
//   int4   symmetric group quantisation along the row (scale = max(absmax / 7, 1e-5), round to
//          nearest even, clamp to [-8, 7]) packed eight values per int32, value i in bits 4i..4i+3
//          stored with the +8 offset of the compressed-tensors "pack-quantized" format;
//   mxfp8  OCP microscaling: groups of 32 along the row share a power-of-two scale (UE8M0 byte,
//          bias 127) chosen as the smallest power of two with absmax / scale <= 448; values are
//          e4m3, saturating.
// (128x128-block fp8 quantisation lives next to the P2P copy kernel that fuses it.)
#include <cuda_fp8.h>

#include "host_utils.h"
#include "ptx.cuh"

namespace axb {

// One warp per (row, group). group in {32, 64, 128}; lanes hold group/32 consecutive values.
template <int GROUP>
__global__ void int4_group_quant_pack_kernel(const __nv_bfloat16* __restrict__ x, int32_t* __restrict__ packed,
                                             __nv_bfloat16* __restrict__ scales, long long rows, int cols,
                                             long long ldx) {
  constexpr int PER = GROUP / 32;           // values per lane (1, 2 or 4)
  const int groups_per_row = cols / GROUP;
  const long long wid = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (wid >= rows * groups_per_row) return;
  const long long r = wid / groups_per_row;
  const int g = static_cast<int>(wid - r * groups_per_row);
  const __nv_bfloat16* src = x + r * ldx + g * GROUP + lane * PER;
  float v[PER];
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    v[i] = __bfloat162float(src[i]);
    amax = fmaxf(amax, fabsf(v[i]));
  }
  amax = warp_max(amax);
  const float scale = fmaxf(amax * (1.0f / 7.0f), 1e-5f);
  uint32_t nib = 0;
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    float q = rintf(__fdiv_rn(v[i], scale));
    q = fminf(fmaxf(q, -8.f), 7.f);
    nib |= (static_cast<uint32_t>(static_cast<int>(q) + 8) & 0xFu) << (4 * i);
  }
  // eight values per int32: gather the nibbles of the 8/PER lanes that share a word
  constexpr int LANES_PER_WORD = 8 / PER;
  uint32_t word = nib << (4 * PER * (lane % LANES_PER_WORD));
#pragma unroll
  for (int o = 1; o < LANES_PER_WORD; o <<= 1) word |= __shfl_xor_sync(0xffffffffu, word, o);
  if (lane % LANES_PER_WORD == 0)
    packed[r * (cols / 8) + (g * GROUP + lane * PER) / 8] = static_cast<int32_t>(word);
  if (lane == 0) scales[r * groups_per_row + g] = __float2bfloat16(scale);
}

// One lane per value, one warp per 32-group.
__global__ void mxfp8_quant_kernel(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ q,
                                   uint8_t* __restrict__ scales, long long rows, int cols, long long ldx) {
  const int groups_per_row = cols / 32;
  const long long wid = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (wid >= rows * groups_per_row) return;
  const long long r = wid / groups_per_row;
  const int g = static_cast<int>(wid - r * groups_per_row);
  const float v = __bfloat162float(x[r * ldx + g * 32 + lane]);
  const float amax = warp_max(fabsf(v));
  int e = -127;                                    // scale 2^e
  if (amax > 0.f && isfinite(amax)) {
    e = static_cast<int>(ceilf(log2f(amax / 448.f)));
    // log2f rounding can leave amax / 2^e a hair above 448: fix up exactly
    if (amax > 448.f * exp2f(static_cast<float>(e))) ++e;
    else if (e > -127 && amax <= 448.f * exp2f(static_cast<float>(e - 1))) --e;
    e = max(-127, min(127, e));
  }
  const float inv = exp2f(static_cast<float>(-e));
  const __nv_fp8_e4m3 f8(v * inv);                 // saturating conversion
  q[r * cols + g * 32 + lane] = *reinterpret_cast<const uint8_t*>(&f8);
  if (lane == 0) scales[r * groups_per_row + g] = static_cast<uint8_t>(e + 127);
}

}  // namespace axb

// x: bf16 [rows][ldx]; packed: int32 [rows][cols/8]; scales: bf16 [rows][cols/group].
extern "C" int axb_int4_group_quant_pack(const void* x, void* packed, void* scales, long long rows, int cols,
                                         long long ldx, int group, void* stream) {
  using namespace axb;
  if (rows <= 0 || cols <= 0 || cols % group != 0 || cols % 8 != 0) return AXB_LAUNCH_BAD_ARG;
  const long long warps = rows * (cols / group);
  const int threads = 256;
  const long long blocks = (warps * 32 + threads - 1) / threads;
  if (blocks > 0x7fffffffLL) return AXB_LAUNCH_TOO_LARGE;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
#define AXB_I4(G)                                                                                      \
  int4_group_quant_pack_kernel<G><<<static_cast<int>(blocks), threads, 0, s>>>(                       \
      static_cast<const __nv_bfloat16*>(x), static_cast<int32_t*>(packed), static_cast<__nv_bfloat16*>(scales), \
      rows, cols, ldx)
  if (group == 32) AXB_I4(32);
  else if (group == 64) AXB_I4(64);
  else if (group == 128) AXB_I4(128);
  else return AXB_LAUNCH_BAD_ARG;
#undef AXB_I4
  return check_launch();
}

// x: bf16 [rows][ldx]; q: e4m3 bytes [rows][cols]; scales: UE8M0 bytes [rows][cols/32].
extern "C" int axb_mxfp8_quant(const void* x, void* q, void* scales, long long rows, int cols, long long ldx,
                               void* stream) {
  using namespace axb;
  if (rows <= 0 || cols <= 0 || cols % 32 != 0) return AXB_LAUNCH_BAD_ARG;
  const long long warps = rows * (cols / 32);
  const int threads = 256;
  const long long blocks = (warps * 32 + threads - 1) / threads;
  if (blocks > 0x7fffffffLL) return AXB_LAUNCH_TOO_LARGE;
  mxfp8_quant_kernel<<<static_cast<int>(blocks), threads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<uint8_t*>(q), static_cast<uint8_t*>(scales), rows, cols, ldx);
  return check_launch();
}
