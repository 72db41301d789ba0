// Split-KV decode attention: the bodies of the range kernel and of the merge step as
// device functions, so that the stand-alone kernels (attention.cu) and the whole-token
// decode kernel (token_kernel.cu) run the same arithmetic in the same order and give
// the same bits.  A "unit" is one KV range of one KV head for NREP query heads, worked
// on by 128 threads that synchronise through `sync` (the CTA barrier in the stand-alone
// kernel, a named barrier of a 4-warp group inside a larger CTA).
// Every file that includes this header is compiled with -fmad=false: a product and a sum
// are only fused where the source says fmaf.
#pragma once

#include "common.cuh"
#include "kernels.h"
#include "quant_device.cuh"

namespace emelb {
namespace fa {

struct CtaSync {
  __device__ __forceinline__ void operator()() const { __syncthreads(); }
};
// named barrier `id` (1..15) for 128 threads
struct GroupSync {
  int id;
  __device__ __forceinline__ void operator()() const { asm volatile("bar.sync %0, 128;" ::"r"(id) : "memory"); }
};

__device__ __forceinline__ void unpack8(const uint4 v, float (&f)[8]) {
  const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __half22float2(h[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}

// reduction over the 128 threads of a unit; tid = thread index inside the unit
template <int NREP, class Sync>
__device__ __forceinline__ void unit_reduce(float (&v)[NREP], float* scratch /*[4][NREP]*/, bool is_max, int tid, Sync sync) {
  const int lane = tid & 31, warp = tid >> 5;
#pragma unroll
  for (int r = 0; r < NREP; ++r) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float t = __shfl_xor_sync(0xffffffffu, v[r], o);
      v[r] = is_max ? fmaxf(v[r], t) : v[r] + t;
    }
    if (lane == 0) scratch[warp * NREP + r] = v[r];
  }
  sync();
#pragma unroll
  for (int r = 0; r < NREP; ++r) {
    float t = scratch[r];
    for (int w = 1; w < 4; ++w) t = is_max ? fmaxf(t, scratch[w * NREP + r]) : t + scratch[w * NREP + r];
    v[r] = t;
  }
  sync();
}

// (K and V rows are read through the non-coherent path: a cache row is written once, by the step of its own
// position, before any unit of that step reads it, and nothing reads it earlier in the same launch; q and the
// partials are rewritten within a launch of the whole-token kernel and bypass L1.)
// One unit: scores for the range (8 lanes per token row, 128-bit loads), exact range
// maximum, probabilities, then the V accumulation with 128-bit loads; f32 throughout.
// s_p: NREP * LMAX floats, s_red: 4 * NREP floats of shared memory owned by the unit.
// T = live token count; ranges are L = ceil(T / splits) tokens (at most LMAX).
// U = token rows a thread loads ahead (register budget of the caller; the results do not depend on it).
// QL2: read q past L1 (the whole-token kernel rewrites q within a launch).
template <int D, int NREP, int LMAX, int U, bool QL2, class Sync>
__device__ __forceinline__ void split_unit(const FlashArgs& a, int split, int kh, int zgroup, int T, int tid, float* s_p,
                                           float* s_red, Sync sync) {
  constexpr int DPL = D / 8;   // dims per lane while scoring (8 lanes per token row)
  constexpr int TPR = D / 8;   // threads per token row while accumulating V (8 halves each)
  constexpr int SLOTS = 128 / TPR;
  // the V reduction reuses the score buffer, SB slots at a time (the order of the additions does not
  // depend on SB)
  constexpr int SB = LMAX / D < SLOTS ? LMAX / D : SLOTS;
  static_assert(SB >= 1 && SLOTS % SB == 0, "slot batches");
  const int n_rep = a.heads / a.kv_heads;
  const int head0 = kh * n_rep + zgroup * NREP;
  int L = (T + a.splits - 1) / a.splits;
  L = L > LMAX ? LMAX : L;  // the host sizes `splits` so this never clips
  const int t0 = split * L;
  const int t1 = min(T, t0 + L);
  const int n = t1 > t0 ? t1 - t0 : 0;

  if (n == 0) {
    for (int idx = tid; idx < NREP * D; idx += 128)
      a.part_acc[((size_t)(head0 + idx / D) * a.splits + split) * D + idx % D] = 0.0f;
    if (tid < NREP) {
      float* ml = a.part_ml + ((size_t)(head0 + tid) * a.splits + split) * 2;
      ml[0] = -INFINITY;
      ml[1] = 0.0f;
    }
    return;
  }

  // pull this range's V rows towards L2 while the scores are computed
  {
    const char* vrange = reinterpret_cast<const char*>(a.v) + (size_t)kh * a.v_nb2 + (size_t)t0 * a.v_nb1;
    const size_t vbytes = (size_t)n * a.v_nb1;
    for (size_t off = (size_t)tid * 128; off < vbytes; off += 128 * 128) asm volatile("prefetch.global.L2 [%0];" ::"l"(vrange + off));
  }
  // ---- scores: q is rounded to f16 first, as the reference does (detail.hpp:5255)
  const int l8 = tid & 7, slot = tid >> 3;
  float q[NREP][DPL];
#pragma unroll
  for (int r = 0; r < NREP; ++r)
#pragma unroll
    for (int i = 0; i < DPL; i += 4) {
      const float4* src = reinterpret_cast<const float4*>(a.q + (size_t)(head0 + r) * D + l8 * DPL + i);
      const float4 t = QL2 ? __ldcg(src) : __ldg(src);
      q[r][i] = __half2float(__float2half_rn(t.x));
      q[r][i + 1] = __half2float(__float2half_rn(t.y));
      q[r][i + 2] = __half2float(__float2half_rn(t.z));
      q[r][i + 3] = __half2float(__float2half_rn(t.w));
    }

  float mx[NREP];
#pragma unroll
  for (int r = 0; r < NREP; ++r) mx[r] = -INFINITY;
  const char* kbase = reinterpret_cast<const char*>(a.k) + (size_t)kh * a.k_nb2 + (size_t)l8 * DPL * 2;
  // the loop bound is uniform across the warp (the score reduction below shuffles
  // over all 32 lanes); rows past the range are clamped on load and masked on store
  for (int tb = 0; tb < n; tb += 16 * U) {
    const int t = tb + slot;
    uint4 kv[U][DPL / 8];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int tt = min(t + 16 * u, n - 1);
      const uint4* kp = reinterpret_cast<const uint4*>(kbase + (size_t)(t0 + tt) * a.k_nb1);
#pragma unroll
      for (int c = 0; c < DPL / 8; ++c) kv[u][c] = __ldg(kp + c);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      float s[NREP];
#pragma unroll
      for (int r = 0; r < NREP; ++r) s[r] = 0.0f;
#pragma unroll
      for (int c = 0; c < DPL / 8; ++c) {
        float kf[8];
        unpack8(kv[u][c], kf);
#pragma unroll
        for (int r = 0; r < NREP; ++r)
#pragma unroll
          for (int i = 0; i < 8; ++i) s[r] = fmaf(q[r][8 * c + i], kf[i], s[r]);
      }
      const int tt = t + 16 * u;
#pragma unroll
      for (int r = 0; r < NREP; ++r) {
        float v = s[r];
        v += __shfl_xor_sync(0xffffffffu, v, 1);
        v += __shfl_xor_sync(0xffffffffu, v, 2);
        v += __shfl_xor_sync(0xffffffffu, v, 4);
        v *= a.scale;
        if (tt < n) {
          mx[r] = fmaxf(mx[r], v);
          if (l8 == 0) s_p[r * LMAX + tt] = v;
        }
      }
    }
  }
  unit_reduce<NREP>(mx, s_red, true, tid, sync);  // also orders the score writes before the reads below

  // ---- probabilities relative to the range maximum
  float lsum[NREP];
#pragma unroll
  for (int r = 0; r < NREP; ++r) lsum[r] = 0.0f;
  for (int idx = tid; idx < n; idx += 128) {
#pragma unroll
    for (int r = 0; r < NREP; ++r) {
      const float pr = expf(s_p[r * LMAX + idx] - mx[r]);
      s_p[r * LMAX + idx] = pr;
      lsum[r] += pr;
    }
  }
  unit_reduce<NREP>(lsum, s_red, false, tid, sync);

  // ---- V accumulation: TPR threads cover one token row with 128-bit loads
  const int c = tid % TPR, vs = tid / TPR;
  float acc[NREP][8];
#pragma unroll
  for (int r = 0; r < NREP; ++r)
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[r][i] = 0.0f;
  const char* vbase = reinterpret_cast<const char*>(a.v) + (size_t)kh * a.v_nb2 + (size_t)c * 16;
  for (int t = vs; t < n; t += SLOTS * U) {
    uint4 vv[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int tt = min(t + SLOTS * u, n - 1);
      vv[u] = __ldg(reinterpret_cast<const uint4*>(vbase + (size_t)(t0 + tt) * a.v_nb1));
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int tt = t + SLOTS * u;
      if (tt < n) {
        float vf[8];
        unpack8(vv[u], vf);
#pragma unroll
        for (int r = 0; r < NREP; ++r) {
          const float pr = s_p[r * LMAX + tt];
#pragma unroll
          for (int i = 0; i < 8; ++i) acc[r][i] = fmaf(pr, vf[i], acc[r][i]);
        }
      }
    }
  }
  sync();  // all probability reads done; the buffer becomes the slot reduction area
  float rsum[(NREP * D + 127) / 128];
#pragma unroll
  for (int j = 0; j < (NREP * D + 127) / 128; ++j) rsum[j] = 0.0f;
#pragma unroll
  for (int sb = 0; sb < SLOTS; sb += SB) {
    if (sb > 0) sync();
    if (vs >= sb && vs < sb + SB) {
#pragma unroll
      for (int r = 0; r < NREP; ++r)
#pragma unroll
        for (int i = 0; i < 8; ++i) s_p[((vs - sb) * NREP + r) * D + c * 8 + i] = acc[r][i];
    }
    sync();
#pragma unroll
    for (int j = 0; j < (NREP * D + 127) / 128; ++j) {
      const int idx = tid + 128 * j;
      if (idx < NREP * D) {
        const int r = idx / D, d = idx % D;
#pragma unroll
        for (int s = 0; s < SB; ++s) rsum[j] += s_p[(s * NREP + r) * D + d];
      }
    }
  }
#pragma unroll
  for (int j = 0; j < (NREP * D + 127) / 128; ++j) {
    const int idx = tid + 128 * j;
    if (idx < NREP * D) a.part_acc[((size_t)(head0 + idx / D) * a.splits + split) * D + idx % D] = rsum[j];
  }
  if (tid < NREP) {
    float* ml = a.part_ml + ((size_t)(head0 + tid) * a.splits + split) * 2;
    ml[0] = mx[tid];
    ml[1] = lsum[tid];
  }
}

// merge of the ranges of one head: out = sum_s e^{m_s-M} acc_s / sum_s e^{m_s-M} l_s.
// One warp turns the head's (max, sum) pairs into weights w[0..63] and 1/denominator ...
constexpr int kMergeMaxSplits = 64;

__device__ __forceinline__ void merge_head_weights(const FlashArgs& a, int head, int lane, float* w /*[64]*/, float* inv) {
  const float* ml = a.part_ml + (size_t)head * a.splits * 2;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.0f, l1 = 0.0f;
  if (lane < a.splits) { m0 = __ldcg(ml + 2 * lane); l0 = __ldcg(ml + 2 * lane + 1); }
  if (lane + 32 < a.splits) { m1 = __ldcg(ml + 2 * (lane + 32)); l1 = __ldcg(ml + 2 * (lane + 32) + 1); }
  float M = fmaxf(m0, m1);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
  const float w0 = m0 == -INFINITY ? 0.0f : expf(m0 - M), w1 = m1 == -INFINITY ? 0.0f : expf(m1 - M);
  w[lane] = w0;
  w[lane + 32] = w1;
  float den = fmaf(w1, l1, w0 * l0);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) den += __shfl_xor_sync(0xffffffffu, den, o);
  if (lane == 0) *inv = den == 0.0f ? 0.0f : 1.0f / den;
}

// ... then every output value walks the ranges in ascending order; the loads of 8 ranges (for each of the
// N values a thread owns) are issued together, the additions keep the order of the ranges
template <int N>
__device__ __forceinline__ void merge_outputs(const FlashArgs& a, const int (&head)[N], const int (&d)[N], const float* const (&w)[N],
                                              const float (&inv)[N], float (&out)[N]) {
  const int D = a.head_dim;
  const float* pa[N];
#pragma unroll
  for (int n = 0; n < N; ++n) {
    pa[n] = a.part_acc + (size_t)head[n] * a.splits * D + d[n];
    out[n] = 0.0f;
  }
  int s = 0;
  for (; s + 8 <= a.splits; s += 8) {
    float v[N][8];
#pragma unroll
    for (int n = 0; n < N; ++n)
#pragma unroll
      for (int k = 0; k < 8; ++k) v[n][k] = __ldcg(pa[n] + (size_t)(s + k) * D);
#pragma unroll
    for (int n = 0; n < N; ++n)
#pragma unroll
      for (int k = 0; k < 8; ++k) out[n] = fmaf(w[n][s + k], v[n][k], out[n]);
  }
  for (; s < a.splits; ++s)
#pragma unroll
    for (int n = 0; n < N; ++n) out[n] = fmaf(w[n][s], __ldcg(pa[n] + (size_t)s * D), out[n]);
#pragma unroll
  for (int n = 0; n < N; ++n) out[n] = out[n] * inv[n];
}

__device__ __forceinline__ float merge_output(const FlashArgs& a, int head, int d, const float* w, float inv) {
  const int h1[1] = {head}, d1[1] = {d};
  const float* const w1[1] = {w};
  const float i1[1] = {inv};
  float o[1];
  merge_outputs<1>(a, h1, d1, w1, i1, o);
  return o[0];
}

}  // namespace fa
}  // namespace emelb
