// expf with the bits of the host C library's expf.
//
// The reference calls libm's expf in two places on this path: silu(gate) in the
// feed-forward (src/emel/text/generator/detail.hpp:2967-2973) and the online
// softmax of flash attention (std::exp(float), src/emel/kernel/detail.hpp:5270-5277).
// Activations are re-quantized to int8 after every such step, so a one-ulp
// difference eventually flips a quantized value and the decode diverges from the
// reference by far more than the logit tolerance.  This function therefore
// restates the published algorithm glibc (>= 2.27) uses for expf — exp(x) =
// 2^(k/32) * 2^(r/32), a 32-entry table of 2^(i/32) and a degree-3 polynomial, all
// in double, rounded once to float (Szabolcs Nagy's expf, ARM optimized-routines) —
// with the operation fusions of glibc's x86-64 FMA build: r and the three
// polynomial steps are single fused multiply-adds.  tests/test_expf_exact.py
// compares it with the host's expf over the float range on the CPU; the same
// source compiles for the device, where double arithmetic is IEEE too.
#pragma once

#include <math.h>
#include <stdint.h>
#include <string.h>

#if defined(__CUDACC__)
#define EMELB_HD __host__ __device__ __forceinline__
#else
#define EMELB_HD static inline
#endif

namespace emelb {

EMELB_HD double expf_bits_to_double(uint64_t u) {
#if defined(__CUDA_ARCH__)
  return __longlong_as_double((long long)u);
#else
  double d;
  memcpy(&d, &u, 8);
  return d;
#endif
}
EMELB_HD uint64_t expf_double_to_bits(double d) {
#if defined(__CUDA_ARCH__)
  return (uint64_t)__double_as_longlong(d);
#else
  uint64_t u;
  memcpy(&u, &d, 8);
  return u;
#endif
}

// 2^(i/32) as IEEE-754 double bits minus (i << 47): adding (k << 47) then lands
// the exponent of 2^(k/32) directly (nearest doubles of 2^(i/32))
#define EMELB_EXPF_TABLE \
  0x3ff0000000000000ull, 0x3fefd9b0d3158574ull, 0x3fefb5586cf9890full, 0x3fef9301d0125b51ull, \
  0x3fef72b83c7d517bull, 0x3fef54873168b9aaull, 0x3fef387a6e756238ull, 0x3fef1e9df51fdee1ull, \
  0x3fef06fe0a31b715ull, 0x3feef1a7373aa9cbull, 0x3feedea64c123422ull, 0x3feece086061892dull, \
  0x3feebfdad5362a27ull, 0x3feeb42b569d4f82ull, 0x3feeab07dd485429ull, 0x3feea47eb03a5585ull, \
  0x3feea09e667f3bcdull, 0x3fee9f75e8ec5f74ull, 0x3feea11473eb0187ull, 0x3feea589994cce13ull, \
  0x3feeace5422aa0dbull, 0x3feeb737b0cdc5e5ull, 0x3feec49182a3f090ull, 0x3feed503b23e255dull, \
  0x3feee89f995ad3adull, 0x3feeff76f2fb5e47ull, 0x3fef199bdd85529cull, 0x3fef3720dcef9069ull, \
  0x3fef5818dcfba487ull, 0x3fef7c97337b9b5full, 0x3fefa4afa2a490daull, 0x3fefd0765b6e4540ull,
static const uint64_t kExpfTable[32] = {EMELB_EXPF_TABLE};
#if defined(__CUDACC__)
// the device's copy lives in global memory (read through L1): lanes index it with different k, and a
// constant-bank or stack copy would serialize or be rebuilt per call
static __device__ const uint64_t kExpfTableDev[32] = {EMELB_EXPF_TABLE};
#endif
#undef EMELB_EXPF_TABLE

EMELB_HD float expf_exact(float x) {
  const float ax = fabsf(x);
  if (!(ax < 88.0f)) {               // |x| >= 88, inf or nan
    if (x != x) return x + x;
    if (x > 0x1.62e42ep6f) return INFINITY;   // overflow (also +inf)
    if (x < -0x1.9fe368p6f) return 0.0f;      // underflow (also -inf)
  }
  const double xd = (double)x;
  const double inv_ln2_n = 0x1.71547652b82fep+0 * 32.0;
  const double shift = 0x1.8p+52;
  const double z = inv_ln2_n * xd;
  double kd = z + shift;             // round to nearest integer, kept in the low mantissa bits
  const uint64_t ki = expf_double_to_bits(kd);
  kd -= shift;
  const double r = fma(inv_ln2_n, xd, -kd);
#if defined(__CUDA_ARCH__)
  uint64_t t = __ldg(&kExpfTableDev[ki & 31]);
#else
  uint64_t t = kExpfTable[ki & 31];
#endif
  t += ki << (52 - 5);
  const double s = expf_bits_to_double(t);
  const double c0 = 0x1.c6af84b912394p-5 / 32.0 / 32.0 / 32.0;
  const double c1 = 0x1.ebfce50fac4f3p-3 / 32.0 / 32.0;
  const double c2 = 0x1.62e42ff0c52d6p-1 / 32.0;
  const double zz = fma(c0, r, c1);
  const double r2 = r * r;
  double y = fma(c2, r, 1.0);
  y = fma(zz, r2, y);
  y = y * s;
  return (float)y;
}

}  // namespace emelb
