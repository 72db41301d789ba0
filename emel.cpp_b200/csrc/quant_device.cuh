// Device-side bodies of the bit-exact activation quantizers, shared by the
// stand-alone quantize kernels and the fused normalisation / activation kernels.
// Every file that includes this header is compiled with -fmad=false; divisions
// use the IEEE round-to-nearest intrinsics.
#pragma once

#include "common.cuh"
#include "kernels.h"

namespace emelb {

// nearest_int, src/emel/kernel/detail.hpp:692-697 (1.5*2^23 magic add)
__device__ __forceinline__ int nearest_int_rn(float v) {
  const float biased = __fadd_rn(v, 12582912.0f);
  return (__float_as_int(biased) & 0x007fffff) - 0x00400000;
}

// quantize_row_q8_k_strided for one 256-block held by a full warp: lane l owns
// elements 8l..8l+7 (src/emel/kernel/detail.hpp:826-867).  Returns the lane's 8
// quants packed in (lo, hi), the 16-wide bsum (valid on even lanes) and d.
__device__ __forceinline__ void q8_k_block_warp(const float (&v)[8], int lane, uint32_t& lo, uint32_t& hi, int& bsum16,
                                                float& d) {
  float amax = 0.0f, mx = 0.0f;
  int idx = 8 * lane;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const float a = fabsf(v[i]);
    if (a > amax) { amax = a; mx = v[i]; idx = 8 * lane + i; }
  }
  // the first element attaining the largest |x| wins (strict > scan in the reference)
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float oa = __shfl_xor_sync(0xffffffffu, amax, o);
    const float om = __shfl_xor_sync(0xffffffffu, mx, o);
    const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
    if (oa > amax || (oa == amax && oi < idx)) { amax = oa; mx = om; idx = oi; }
  }
  int q[8];
  d = 0.0f;
  if (amax == 0.0f) {
#pragma unroll
    for (int i = 0; i < 8; ++i) q[i] = 0;
  } else {
    const float iscale = __fdiv_rn(-127.0f, mx);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int t = nearest_int_rn(__fmul_rn(iscale, v[i]));
      q[i] = (int)(int8_t)(t < 127 ? t : 127);
    }
    d = __fdiv_rn(1.0f, iscale);
  }
  int s = 0;
#pragma unroll
  for (int i = 0; i < 8; ++i) s += q[i];
  bsum16 = s + __shfl_xor_sync(0xffffffffu, s, 1);
  lo = 0;
  hi = 0;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    lo |= (uint32_t)(q[i] & 0xff) << (8 * i);
    hi |= (uint32_t)(q[4 + i] & 0xff) << (8 * i);
  }
}

__device__ __forceinline__ void q8_k_store_planes(const ActPlanesMut& p, int col, int K, int blk, int lane, uint32_t lo,
                                                  uint32_t hi, int bsum16, float d) {
  const int64_t e0 = (int64_t)blk * QK_K + 8 * lane;
  *reinterpret_cast<uint2*>(p.qs + (int64_t)col * K + e0) = make_uint2(lo, hi);
  if ((lane & 1) == 0) p.bsums[(int64_t)col * (K / 16) + blk * 16 + (lane >> 1)] = (int16_t)bsum16;
  if (lane == 0) p.d[(int64_t)col * (K / QK_K) + blk] = d;
}

// quantize_row_q8_0_strided for one 32-block held by 8 consecutive lanes, 4
// elements per lane (src/emel/kernel/detail.hpp:804-824; std::round = roundf).
// Returns the 4 packed quants and the f16-rounded scale.
__device__ __forceinline__ void q8_0_block_oct(const float (&v)[4], uint32_t& w, __half& dh) {
  float amax = 0.0f;
#pragma unroll
  for (int i = 0; i < 4; ++i) amax = fmaxf(amax, fabsf(v[i]));
#pragma unroll
  for (int o = 4; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  const float d = __fdiv_rn(amax, 127.0f);
  const float id = d != 0.0f ? __fdiv_rn(1.0f, d) : 0.0f;
  w = 0;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    int t = (int)roundf(__fmul_rn(v[i], id));
    t = t < -127 ? -127 : (t > 127 ? 127 : t);
    w |= (uint32_t)(t & 0xff) << (8 * i);
  }
  dh = __float2half_rn(d);  // fp32_to_fp16, src/emel/kernel/detail.hpp:372-392 (RNE)
}

}  // namespace emelb
