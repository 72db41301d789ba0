// Q4_K x Q8_K mat-vec building blocks of the whole-token decode kernel
// (token_kernel.cu).
//
// What differs from the stand-alone streaming kernel (gemv2.cu):
//   * an item is a group of 4*R rows x 2048 weights and items are independent:
//     the per-block float values of a row (fma(d*dx, isum, -(dmin*dx)*msum), the
//     reference's x86 route, src/emel/kernel/x86_64/actions.hpp:859-866) go to a
//     scratch table and the warp that completes a row group adds them up in
//     ascending block order (:876-896), so the result does not depend on which
//     warp computed which chunk and short, wide matrices (down projection) spread
//     over the whole machine;
//   * a lane decodes R blocks that share one activation span: the 16 activation
//     loads of a span serve R rows;
//   * every shared-memory access is an explicit ld.shared with a 32-bit address
//     (one LOP3 per swizzled activation address, immediates for the weights);
//   * the min term is four dp2a over pre-added 32-element activation sums, the
//     high-nibble dots stay scaled by 16 until the end of the block;
//   * the row chunks of an item are copied by 4*R lanes, one bulk copy each, in
//     one SIMT pass.
#pragma once

#include "common.cuh"
#include "kernels.h"
#include "quant_device.cuh"

namespace emelb {
namespace g4 {

constexpr int CHUNK = 2048;             // weights of one row in an item
constexpr int CB = 8 * Q4_K_BYTES;      // 1152 bytes: one row's share of an item
constexpr int kWaitPolls = 1 << 22;
constexpr unsigned long long kWaitNs = 1000000000ull;  // 1 s

__device__ __forceinline__ uint32_t s32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint32_t bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// bounded twice: by poll count and by wall time (a poll may itself block for a while)
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity) {
  int spins = 0;
  bool ok = false;
  unsigned long long t_start = 0;
  while (!(ok = mbar_try_wait(bar, parity)) && ++spins < kWaitPolls) {
    if ((spins & 255) == 0) {
      unsigned long long now;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
      if (t_start == 0) t_start = now;
      else if (now - t_start > kWaitNs) break;
    }
  }
  return ok;
}
// global -> this CTA's shared memory, completion counted in bytes on `bar`;
// both addresses 16-byte aligned, size a multiple of 16
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src),
               "r"(bytes), "r"(bar)
               : "memory");
}

__device__ __forceinline__ void lds128(uint32_t addr, uint32_t* v) {
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]) : "r"(addr));
}
__device__ __forceinline__ float lds_f32(uint32_t addr) {
  float v;
  asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ int dp4a_us(uint32_t a_unsigned, int b_signed, int c) {
  int d;
  asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a_unsigned), "r"(b_signed), "r"(c));
  return d;
}
// c + s16(a.lo) * u8(b.byte0|2) + s16(a.hi) * u8(b.byte1|3)
__device__ __forceinline__ int dp2a_lo(uint32_t pair, uint32_t bytes, int c) {
  int d;
  asm("dp2a.lo.s32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(pair), "r"(bytes), "r"(c));
  return d;
}
__device__ __forceinline__ int dp2a_hi(uint32_t pair, uint32_t bytes, int c) {
  int d;
  asm("dp2a.hi.s32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(pair), "r"(bytes), "r"(c));
  return d;
}

// ---------------------------------------------------------------- activations in shared memory
// One quantized activation vector (Q8_K numbers) as the item code reads it, at a
// 256-byte aligned shared address A:
//   A                 K int8; the 16-byte units of every 256-byte span s are kept at
//                     unit ^ (s & 7): the 8 lanes of a row read the same unit of 8
//                     consecutive spans at once and would otherwise share a bank group
//   A + K             K/256 x 8 int16: sums of the 8 runs of 32 quants of each block
//   A + K + K/16      K/256 f32 block scales
__host__ __device__ constexpr int act_bytes(int K) { return ((K + K / 16 + K / 64) + 255) & ~255; }

// copy from the quantized planes (qs / d / bsums of one column); all threads of the CTA
__device__ __forceinline__ void stage_act_planes(uint8_t* A, int K, const int8_t* qs, const float* d, const int16_t* bsums,
                                                 int tid, int nthreads) {
  const int4* gq = reinterpret_cast<const int4*>(qs);
  int4* sq = reinterpret_cast<int4*>(A);
  for (int i = tid; i < K / 16; i += nthreads) sq[i ^ ((i >> 4) & 7)] = __ldcg(gq + i);
  uint4* sp = reinterpret_cast<uint4*>(A + K);
  const int4* gb = reinterpret_cast<const int4*>(bsums);
  float* sd = reinterpret_cast<float*>(A + K + K / 16);
  for (int blk = tid; blk < K / QK_K; blk += nthreads) {
    const int4 b0 = __ldcg(gb + 2 * blk), b1 = __ldcg(gb + 2 * blk + 1);
    const int w[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int p0 = (int)(short)(w[2 * j] & 0xffff) + (w[2 * j] >> 16);
      const int p1 = (int)(short)(w[2 * j + 1] & 0xffff) + (w[2 * j + 1] >> 16);
      o[j] = (uint32_t)(p0 & 0xffff) | ((uint32_t)p1 << 16);
    }
    sp[blk] = make_uint4(o[0], o[1], o[2], o[3]);
    sd[blk] = __ldcg(d + blk);
  }
}

struct CtaBarrier {
  __device__ __forceinline__ void operator()() const { __syncthreads(); }
};

// One Q8_K block (256 values, 8 per lane) quantized by a warp into the shared activation vector
// (quantizer: src/emel/kernel/detail.hpp:826-867)
__device__ __forceinline__ void stage_block(uint8_t* A, int K, int blk, int lane, const float (&v)[8]) {
  uint32_t lo, hi;
  int bs16;
  float dq;
  q8_k_block_warp(v, lane, lo, hi, bs16, dq);
  const int unit = blk * 16 + ((lane >> 1) ^ (blk & 7));
  *reinterpret_cast<uint2*>(A + unit * 16 + (lane & 1) * 8) = make_uint2(lo, hi);
  const int ps = bs16 + __shfl_xor_sync(0xffffffffu, bs16, 2);   // lanes 4j and 4j+2 hold the two halves of run j
  if ((lane & 3) == 0) reinterpret_cast<int16_t*>(A + K)[blk * 8 + (lane >> 2)] = (int16_t)ps;
  if (lane == 0) reinterpret_cast<float*>(A + K + K / 16)[blk] = dq;
}

// out = (x * 1/sqrt(mean(x^2) + eps)) * w quantized to Q8_K straight into shared memory
// (rms_norm: src/emel/text/generator/detail.hpp:2735-2756, f64 sum of the f32 squares).
// The WARPS warps that call it synchronise through `sync` (their common barrier); s_part holds one double per
// warp.  Warp w owns blocks w, w + WARPS, ...: up to BPW blocks stay in registers between the sum of squares
// and the scaling (one pass over x); longer vectors are read twice.
template <int WARPS, class Sync>
__device__ __forceinline__ void stage_act_rms_norm(uint8_t* A, int K, const float* x, const float* w, float eps, double* s_part,
                                                   int warp, int lane, Sync sync) {
  constexpr int BPW = 2;
  const int nblk = K / QK_K;
  const bool in_regs = nblk <= BPW * WARPS;
  float xv[BPW][8];
  double ss = 0.0;
  if (in_regs) {
#pragma unroll
    for (int j = 0; j < BPW; ++j) {
      const int blk = warp + j * WARPS;
      if (blk < nblk) {
        const float4* src = reinterpret_cast<const float4*>(x + blk * QK_K + 8 * lane);
        const float4 x0 = __ldcg(src), x1 = __ldcg(src + 1);
        xv[j][0] = x0.x; xv[j][1] = x0.y; xv[j][2] = x0.z; xv[j][3] = x0.w;
        xv[j][4] = x1.x; xv[j][5] = x1.y; xv[j][6] = x1.z; xv[j][7] = x1.w;
#pragma unroll
        for (int i = 0; i < 8; ++i) ss += (double)__fmul_rn(xv[j][i], xv[j][i]);
      }
    }
  } else {
    for (int i = warp * 32 + lane; i < K; i += WARPS * 32) {
      const float v = __ldcg(x + i);
      ss += (double)__fmul_rn(v, v);
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  sync();   // s_part may still be read by a previous use
  if (lane == 0) s_part[warp] = ss;
  sync();
  double total = 0.0;
#pragma unroll
  for (int i = 0; i < WARPS; ++i) total += s_part[i];
  const float mean = (float)(total / (double)K);
  const float scale = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(mean, eps)));
  for (int j = 0; warp + j * WARPS < nblk; ++j) {
    const int blk = warp + j * WARPS;
    const int e0 = blk * QK_K + 8 * lane;
    float xs[8];
    if (in_regs) {
#pragma unroll
      for (int jj = 0; jj < BPW; ++jj)
        if (jj == j) {
#pragma unroll
          for (int i = 0; i < 8; ++i) xs[i] = xv[jj][i];
        }
    } else {
      const float4 x0 = __ldcg(reinterpret_cast<const float4*>(x + e0)), x1 = __ldcg(reinterpret_cast<const float4*>(x + e0) + 1);
      xs[0] = x0.x; xs[1] = x0.y; xs[2] = x0.z; xs[3] = x0.w; xs[4] = x1.x; xs[5] = x1.y; xs[6] = x1.z; xs[7] = x1.w;
    }
    const float4 w0 = __ldg(reinterpret_cast<const float4*>(w + e0)), w1 = __ldg(reinterpret_cast<const float4*>(w + e0) + 1);
    const float ws[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
    float v[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = __fmul_rn(__fmul_rn(xs[i], scale), ws[i]);
    stage_block(A, K, blk, lane, v);
  }
}

// x (f32) quantized to Q8_K into shared memory, no normalisation; warp w owns blocks w, w + WARPS, ...
template <int WARPS>
__device__ __forceinline__ void stage_act_f32(uint8_t* A, int K, const float* x, int warp, int lane) {
  for (int blk = warp; blk < K / QK_K; blk += WARPS) {
    const float4* src = reinterpret_cast<const float4*>(x + blk * QK_K + 8 * lane);
    const float4 x0 = __ldcg(src), x1 = __ldcg(src + 1);
    const float v[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
    stage_block(A, K, blk, lane, v);
  }
}

// ---------------------------------------------------------------- one item
// Lane (r4 = lane / 8, b = lane % 8) decodes span b (256 weights) of rows r4 + 4*i,
// i < R, of the item staged at `stage` (4*R rows x 1152 bytes); `A` is the 256-byte
// aligned shared address of the activation vector, `blk` = chunk * 8 + b the block
// index inside the row.  bv[i] = the block's value, the float the reference's x86
// route adds to the row sum for this block.
template <int R>
__device__ __forceinline__ void q4k_item(uint32_t stage, uint32_t A, int K, int blk, int lane, float (&bv)[R]) {
  const int r4 = lane >> 3, b = lane & 7;
  const uint32_t wb = stage + r4 * CB + b * Q4_K_BYTES;
  const uint32_t aq = A + blk * 256;
  const uint32_t swb = (uint32_t)b << 4;
  constexpr int RS = 4 * CB;   // rows r4 and r4 + 4 are 4 row slots apart
  uint32_t sc_lo[R], sc_hi[R], mn_lo[R], mn_hi[R], dd[R];
#pragma unroll
  for (int i = 0; i < R; ++i) {
    uint32_t h[4];
    lds128(wb + i * RS, h);
    // get_scale_min_k4 through the kmask word shuffle (src/emel/kernel/x86_64/actions.hpp:793-801)
    dd[i] = h[0];
    sc_lo[i] = h[1] & 0x3f3f3f3fu;
    mn_lo[i] = h[2] & 0x3f3f3f3fu;
    sc_hi[i] = (h[3] & 0x0f0f0f0fu) | (((h[1] >> 6) & 0x03030303u) << 4);
    mn_hi[i] = ((h[3] >> 4) & 0x0f0f0f0fu) | (((h[2] >> 6) & 0x03030303u) << 4);
  }
  int il[R], ih[R];
#pragma unroll
  for (int i = 0; i < R; ++i) { il[i] = 0; ih[i] = 0; }
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    uint32_t a[16];
#pragma unroll
    for (int u = 0; u < 4; ++u) lds128(aq | ((uint32_t)(64 * r + 16 * u) ^ swb), a + 4 * u);
#pragma unroll
    for (int i = 0; i < R; ++i) {
      uint32_t v[8];
      lds128(wb + i * RS + 16 + 32 * r, v);
      lds128(wb + i * RS + 32 + 32 * r, v + 4);
      int lo = 0, hi = 0;
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        lo = __dp4a((int)(v[k] & 0x0f0f0f0fu), (int)a[k], lo);
        hi = dp4a_us(v[k] & 0xf0f0f0f0u, (int)a[8 + k], hi);   // 16 x the high-nibble dot
      }
      const uint32_t scw = r < 2 ? sc_lo[i] : sc_hi[i];
      const int sh = 16 * (r & 1);
      il[i] += (int)((scw >> sh) & 0xffu) * lo;
      ih[i] += (int)((scw >> (sh + 8)) & 0xffu) * hi;
    }
  }
  uint32_t pw[4];
  lds128(A + K + blk * 16, pw);
  const float dx = lds_f32(A + K + K / 16 + blk * 4);
#pragma unroll
  for (int i = 0; i < R; ++i) {
    int ms = dp2a_lo(pw[0], mn_lo[i], 0);
    ms = dp2a_hi(pw[1], mn_lo[i], ms);
    ms = dp2a_lo(pw[2], mn_hi[i], ms);
    ms = dp2a_hi(pw[3], mn_hi[i], ms);
    const int isum = il[i] + (ih[i] >> 4);
    const float d = h2f((uint16_t)(dd[i] & 0xffffu)), dmin = h2f((uint16_t)(dd[i] >> 16));
    bv[i] = __fmaf_rn(__fmul_rn(dx, d), (float)isum, -__fmul_rn(__fmul_rn(dx, dmin), (float)ms));
  }
}

// the 4*R row chunks of one item, one bulk copy per lane < 4*R; rows past the matrix are
// clamped to its last row (their results are dropped)
template <int R>
__device__ __forceinline__ void issue_item(uint32_t stage, uint32_t bar, const uint8_t* W, int64_t row_bytes, int M, int row0,
                                           int chunk, int lane) {
  if (lane == 0) mbar_expect_tx(bar, 4 * R * CB);
  if (lane < 4 * R) {
    const int row = min(row0 + lane, M - 1);
    bulk_g2s(stage + lane * CB, W + (size_t)row * row_bytes + (size_t)chunk * CB, CB, bar);
  }
}

// The item's block values go to the table (row-major, K/256 floats per row, row groups of 4*R rows) ...
template <int R>
__device__ __forceinline__ void store_item(const float (&bv)[R], float* table, int group, int chunk, int nchunks, int lane) {
  const int r4 = lane >> 3, b = lane & 7, nblk = nchunks * 8;
  float* rows = table + (size_t)group * (4 * R) * nblk;
#pragma unroll
  for (int i = 0; i < R; ++i) __stcg(rows + (size_t)(r4 + 4 * i) * nblk + chunk * 8 + b, bv[i]);
}

// ... and the warp that makes the `target`-th arrival for a row group (after its own store_item calls) returns
// true with `sum` = the row's total in ascending block order on lanes < 4*R (lane = row inside the group).
// `cnt` is the group's arrival counter: zero before the first arrival, zero again afterwards.
template <int R>
__device__ __forceinline__ bool arrive_group(const float* table, int* cnt, int group, int target, int nchunks, int lane,
                                             float& sum) {
  const int nblk = nchunks * 8;
  __threadfence();
  __syncwarp();
  int last = 0;
  if (lane == 0) last = atomicAdd(cnt + group, 1) == target - 1;
  last = __shfl_sync(0xffffffffu, last, 0);
  if (!last) return false;
  if (lane == 0) cnt[group] = 0;
  __threadfence();
  sum = 0.0f;
  if (lane < 4 * R) {
    const float4* src = reinterpret_cast<const float4*>(table + ((size_t)group * (4 * R) + lane) * nblk);
#pragma unroll 2
    for (int q = 0; q < nblk / 4; ++q) {
      const float4 t = __ldcg(src + q);
      sum = __fadd_rn(sum, t.x);
      sum = __fadd_rn(sum, t.y);
      sum = __fadd_rn(sum, t.z);
      sum = __fadd_rn(sum, t.w);
    }
  }
  return true;
}

template <int R>
__device__ __forceinline__ bool finish_item(const float (&bv)[R], float* table, int* cnt, int group, int chunk, int nchunks,
                                            int lane, float& sum) {
  store_item<R>(bv, table, group, chunk, nchunks, lane);
  return arrive_group<R>(table, cnt, group, nchunks, nchunks, lane, sum);
}

}  // namespace g4
}  // namespace emelb
