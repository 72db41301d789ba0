// Decode GEMV / small-batch GEMM over GGUF block-quantized weight rows:
//   y[i*ldy + j] = sum_k W[i][k] * x_j[k]        (W: Q4_K | Q6_K | Q8_0 | Q4_0,
//                                                 x_j: Q8_K / Q8_0 planes)
// Replaces the row-dot loops of the reference's op_mul_mat
// (src/emel/kernel/detail.hpp:2846-2942, 3062-3153, 3252-3269, 3356-3571;
//  src/emel/kernel/x86_64/actions.hpp:763-1107, 1186-1326).
//
// HBM-bound design.  The weight matrix is streamed exactly once as 2048-element
// row chunks (a multiple of 16 bytes for all four block formats: 1152 / 1680 /
// 2176 / 1152 B).  Every warp owns a private ring of shared-memory stages and
// fills it with 16-byte cp.async copies (fully coalesced whatever the block
// alignment: Q8_0 / Q6_K / Q4_0 blocks sit at 2-byte offsets, so lanes realign
// words out of shared memory with funnel shifts instead of issuing narrow global
// loads).  No block-wide barrier exists in the kernel: a warp only waits on its
// own copies (cp.async.wait_group + __syncwarp), so up to STAGES-1 chunks per
// warp stay in flight while a chunk is consumed.  Per chunk a lane owns 64
// consecutive weights: it unpacks nibbles / 6-bit values in registers, runs
// dp4a integer dots per 16/32-wide sub-block and applies the sub-block scales
// and mins as integers.  A task is R consecutive rows so that one activation
// register set serves R rows.
//
// Float order.  The integers of a block are exact whatever the order, so lanes
// first reduce them per block; the f32 part then follows the reference's x86
// route literally: one value per block — fma(d*dx, isum, -(dmin*dx)*msum) for
// Q4_K, (d*dx)*isum for Q6_K, sumi*(dw*dx) for Q8_0/Q4_0 — added to the row sum
// block after block in ascending order (dot_*_row_avx2_fma,
// src/emel/kernel/x86_64/actions.hpp:876-896, 899-927, 999-1027, 1087-1107).
// For the K-quants the 8 block values of a chunk are walked with shuffles; for
// the 32-wide formats (64 blocks per chunk) they are parked in shared memory and
// one lane per (row, column) walks them.  The result equals the reference's
// AVX2 output bit for bit (and its scalar output for Q8_0/Q4_0, whose two routes
// agree).
#include <cstdlib>

#include "common.cuh"
#include "kernels.h"

namespace emelb {

namespace {

constexpr int CHUNK = 2048;  // weights per row per pipeline item

template <int T> struct Geo;
template <> struct Geo<T_Q4_K> { static constexpr int CB = 8 * Q4_K_BYTES; };
template <> struct Geo<T_Q6_K> { static constexpr int CB = 8 * Q6_K_BYTES; };
template <> struct Geo<T_Q8_0> { static constexpr int CB = 64 * Q8_0_BYTES; };
template <> struct Geo<T_Q4_0> { static constexpr int CB = 64 * Q4_0_BYTES; };

__device__ __forceinline__ uint32_t lds32(const uint8_t* p) { return *reinterpret_cast<const uint32_t*>(p); }

// 16 bytes starting at a 2-byte-aligned shared-memory offset, as 4 words
__device__ __forceinline__ void lds16_unaligned(const uint8_t* base, int off, uint32_t (&out)[4]) {
  const uint8_t* p = base + (off & ~3);
  const int sh = (off & 2) * 8;
  uint32_t w[5];
#pragma unroll
  for (int i = 0; i < 5; ++i) w[i] = lds32(p + 4 * i);
#pragma unroll
  for (int i = 0; i < 4; ++i) out[i] = __funnelshift_r(w[i], w[i + 1], sh);
}

// ---------------------------------------------------------------- activations
template <int T> struct ARegs;

// Q8_K planes, the 64 activations a lane pairs with its 64 weights
template <> struct ARegs<T_Q4_K> {
  int a[16];
  int bs0, bs1;  // bsums of the two 32-wide sub-blocks
  float d;
  __device__ __forceinline__ void load(const ActPlanes& act, int col, int chunk, int lane) {
    const int64_t e0 = (int64_t)chunk * CHUNK + 64 * lane;
    const int4* q = reinterpret_cast<const int4*>(act.qs + col * act.col_stride_qs + e0);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int4 v = __ldg(q + i);
      a[4 * i + 0] = v.x; a[4 * i + 1] = v.y; a[4 * i + 2] = v.z; a[4 * i + 3] = v.w;
    }
    const short4 b = __ldg(reinterpret_cast<const short4*>(act.bsums + col * act.col_stride_bs + e0 / 16));
    bs0 = (int)b.x + (int)b.y;
    bs1 = (int)b.z + (int)b.w;
    d = __ldg(act.d + col * act.col_stride_d + e0 / QK_K);
  }
};

template <> struct ARegs<T_Q6_K> {
  int a[16];     // four 16-wide groups: elements e, e+32, e+64, e+96
  int bs[4];
  float d;
  __device__ __forceinline__ void load(const ActPlanes& act, int col, int chunk, int lane) {
    const int b = lane >> 2, qd = lane & 3;
    const int64_t e0 = (int64_t)chunk * CHUNK + 256 * b + 128 * (qd >> 1) + 16 * (qd & 1);
    const int8_t* q = act.qs + col * act.col_stride_qs + e0;
    const int16_t* s = act.bsums + col * act.col_stride_bs + e0 / 16;
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      const int4 v = __ldg(reinterpret_cast<const int4*>(q + 32 * g));
      a[4 * g + 0] = v.x; a[4 * g + 1] = v.y; a[4 * g + 2] = v.z; a[4 * g + 3] = v.w;
      bs[g] = (int)__ldg(s + 2 * g);
    }
    d = __ldg(act.d + col * act.col_stride_d + e0 / QK_K);
  }
};

// Q8_0 planes: two 32-blocks per lane
struct ARegs32 {
  int a[16];
  float d0, d1;
  __device__ __forceinline__ void load(const ActPlanes& act, int col, int chunk, int lane) {
    const int64_t e0 = (int64_t)chunk * CHUNK + 64 * lane;
    const int4* q = reinterpret_cast<const int4*>(act.qs + col * act.col_stride_qs + e0);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int4 v = __ldg(q + i);
      a[4 * i + 0] = v.x; a[4 * i + 1] = v.y; a[4 * i + 2] = v.z; a[4 * i + 3] = v.w;
    }
    const float2 dd = __ldg(reinterpret_cast<const float2*>(act.d + col * act.col_stride_d + e0 / 32));
    d0 = dd.x;
    d1 = dd.y;
  }
};
template <> struct ARegs<T_Q8_0> : ARegs32 {};
template <> struct ARegs<T_Q4_0> : ARegs32 {};

// ---------------------------------------------------------------- weights
template <int T> struct WRegs;

// Q4_K: lane = (block b = lane/4, 64-element run r = lane%4); the run's 32 bytes
// hold sub-block 2r in the low nibbles and 2r+1 in the high nibbles
// (src/emel/kernel/detail.hpp:533-550); scales/mins per get_scale_min_k4 (:475-485)
template <> struct WRegs<T_Q4_K> {
  uint32_t q[8];
  int sc0, sc1, m0, m1;
  float d, dmin;
  __device__ __forceinline__ void load(const uint8_t* sw, int lane) {
    const uint8_t* blk = sw + Q4_K_BYTES * (lane >> 2);
    const int r = lane & 3;
    const uint4 v0 = *reinterpret_cast<const uint4*>(blk + 16 + 32 * r);
    const uint4 v1 = *reinterpret_cast<const uint4*>(blk + 32 + 32 * r);
    q[0] = v0.x; q[1] = v0.y; q[2] = v0.z; q[3] = v0.w;
    q[4] = v1.x; q[5] = v1.y; q[6] = v1.z; q[7] = v1.w;
    const uint32_t dd = lds32(blk);
    d = h2f((uint16_t)(dd & 0xffffu));
    dmin = h2f((uint16_t)(dd >> 16));
    const uint8_t* s = blk + 4;
    const int j0 = 2 * r, j1 = 2 * r + 1;
    if (r < 2) {
      sc0 = s[j0] & 63; m0 = s[j0 + 4] & 63;
      sc1 = s[j1] & 63; m1 = s[j1 + 4] & 63;
    } else {
      sc0 = (s[j0 + 4] & 0x0f) | ((s[j0 - 4] >> 6) << 4);
      m0 = (s[j0 + 4] >> 4) | ((s[j0] >> 6) << 4);
      sc1 = (s[j1 + 4] & 0x0f) | ((s[j1 - 4] >> 6) << 4);
      m1 = (s[j1 + 4] >> 4) | ((s[j1] >> 6) << 4);
    }
  }
  // value of the lane's block (identical on its 4 lanes):
  // fma(d_all, isum, -d_min * msum), src/emel/kernel/x86_64/actions.hpp:859-866
  __device__ __forceinline__ float block_value(const ARegs<T_Q4_K>& x) const {
    int lo = 0, hi = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      lo = __dp4a((int)(q[i] & 0x0f0f0f0fu), x.a[i], lo);
      hi = __dp4a((int)((q[i] >> 4) & 0x0f0f0f0fu), x.a[8 + i], hi);
    }
    int isum = sc0 * lo + sc1 * hi;
    int msum = m0 * x.bs0 + m1 * x.bs1;
    isum += __shfl_xor_sync(0xffffffffu, isum, 1);
    msum += __shfl_xor_sync(0xffffffffu, msum, 1);
    isum += __shfl_xor_sync(0xffffffffu, isum, 2);
    msum += __shfl_xor_sync(0xffffffffu, msum, 2);
    const float d_all = __fmul_rn(x.d, d), d_min = __fmul_rn(x.d, dmin);
    return __fmaf_rn(d_all, (float)isum, -__fmul_rn(d_min, (float)msum));
  }
};

// Q6_K: lane = (block b = lane/4, half n = (lane%4)/2, 16 positions l0 = 16*(lane%2));
// value = (ql nibble | qh 2 bits << 4) - 32, int8 scale per 16
// (src/emel/kernel/detail.hpp:592-629).  The -32 is applied through the
// activation block sums: sum((u-32)*a) = sum(u*a) - 32*bsum (the identity the
// reference's AVX2 route uses, src/emel/kernel/x86_64/actions.hpp:1036-1076).
template <> struct WRegs<T_Q6_K> {
  uint32_t v[16];  // four 16-wide groups of unsigned 6-bit values
  int sc[4];
  float d;
  __device__ __forceinline__ void load(const uint8_t* sw, int lane) {
    const int off = Q6_K_BYTES * (lane >> 2);
    const int qd = lane & 3, n = qd >> 1, l0 = 16 * (qd & 1);
    uint32_t qa[4], qb[4], qh[4];
    lds16_unaligned(sw, off + 64 * n + l0, qa);
    lds16_unaligned(sw, off + 64 * n + 32 + l0, qb);
    lds16_unaligned(sw, off + 128 + 32 * n + l0, qh);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      v[i] = (qa[i] & 0x0f0f0f0fu) | ((qh[i] & 0x03030303u) << 4);
      v[4 + i] = (qb[i] & 0x0f0f0f0fu) | (((qh[i] >> 2) & 0x03030303u) << 4);
      v[8 + i] = ((qa[i] >> 4) & 0x0f0f0f0fu) | (((qh[i] >> 4) & 0x03030303u) << 4);
      v[12 + i] = ((qb[i] >> 4) & 0x0f0f0f0fu) | (((qh[i] >> 6) & 0x03030303u) << 4);
    }
    const int8_t* s = reinterpret_cast<const int8_t*>(sw + off + 192 + 8 * n + (qd & 1));
#pragma unroll
    for (int g = 0; g < 4; ++g) sc[g] = s[2 * g];
    d = h2f(*reinterpret_cast<const uint16_t*>(sw + off + 208));
  }
  // (dx * d) * (isum - 32 * sum_mins), src/emel/kernel/x86_64/actions.hpp:1073-1077
  __device__ __forceinline__ float block_value(const ARegs<T_Q6_K>& x) const {
    int isum = 0;
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      int s = 0;
#pragma unroll
      for (int i = 0; i < 4; ++i) s = __dp4a((int)v[4 * g + i], x.a[4 * g + i], s);
      isum += sc[g] * (s - 32 * x.bs[g]);
    }
    isum += __shfl_xor_sync(0xffffffffu, isum, 1);
    isum += __shfl_xor_sync(0xffffffffu, isum, 2);
    return __fmul_rn(__fmul_rn(x.d, d), (float)isum);
  }
};

// Q8_0: lane owns blocks 2*lane and 2*lane+1 = 68 bytes at a 4-byte-aligned
// offset; the first block's quants start 2 bytes in and are realigned by shifts
template <> struct WRegs<T_Q8_0> {
  int q0[8], q1[8];
  float d0, d1;
  __device__ __forceinline__ void load(const uint8_t* sw, int lane) {
    const uint8_t* p = sw + 68 * lane;
    uint32_t w[17];
#pragma unroll
    for (int i = 0; i < 17; ++i) w[i] = lds32(p + 4 * i);
    d0 = h2f((uint16_t)(w[0] & 0xffffu));
    d1 = h2f((uint16_t)(w[8] >> 16));
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      q0[i] = (int)__funnelshift_r(w[i], w[i + 1], 16);
      q1[i] = (int)w[9 + i];
    }
  }
  // per block: (float)sumi * (h(dw) * h(dx)), src/emel/kernel/detail.hpp:3257-3266
  __device__ __forceinline__ float2 block_values(const ARegs<T_Q8_0>& x) const {
    int s0 = 0, s1 = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      s0 = __dp4a(q0[i], x.a[i], s0);
      s1 = __dp4a(q1[i], x.a[8 + i], s1);
    }
    return make_float2(__fmul_rn((float)s0, __fmul_rn(d0, x.d0)), __fmul_rn((float)s1, __fmul_rn(d1, x.d1)));
  }
};

// Q4_0: lane owns blocks 2*lane, 2*lane+1 = 36 bytes; element j = low nibble of
// byte j, element j+16 = high nibble, value = nibble - 8
// (src/emel/kernel/detail.hpp:487-502, 3131-3153); the -8 goes through the
// activation sum: sum((u-8)*a) = sum(u*a) - 8*sum(a)
template <> struct WRegs<T_Q4_0> {
  uint32_t q0[4], q1[4];
  float d0, d1;
  __device__ __forceinline__ void load(const uint8_t* sw, int lane) {
    const uint8_t* p = sw + 36 * lane;
    uint32_t w[9];
#pragma unroll
    for (int i = 0; i < 9; ++i) w[i] = lds32(p + 4 * i);
    d0 = h2f((uint16_t)(w[0] & 0xffffu));
    d1 = h2f((uint16_t)(w[4] >> 16));
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      q0[i] = __funnelshift_r(w[i], w[i + 1], 16);
      q1[i] = w[5 + i];
    }
  }
  __device__ __forceinline__ float2 block_values(const ARegs<T_Q4_0>& x) const {
    int s0 = 0, s1 = 0, t0 = 0, t1 = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      s0 = __dp4a((int)(q0[i] & 0x0f0f0f0fu), x.a[i], s0);
      s0 = __dp4a((int)((q0[i] >> 4) & 0x0f0f0f0fu), x.a[4 + i], s0);
      s1 = __dp4a((int)(q1[i] & 0x0f0f0f0fu), x.a[8 + i], s1);
      s1 = __dp4a((int)((q1[i] >> 4) & 0x0f0f0f0fu), x.a[12 + i], s1);
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      t0 = __dp4a(0x01010101, x.a[i], t0);
      t1 = __dp4a(0x01010101, x.a[8 + i], t1);
    }
    return make_float2(__fmul_rn((float)(s0 - 8 * t0), __fmul_rn(d0, x.d0)),
                       __fmul_rn((float)(s1 - 8 * t1), __fmul_rn(d1, x.d1)));
  }
};

// ---------------------------------------------------------------- streaming kernel
constexpr int CHAIN_ROW = 68;  // 64 block values of a chunk + padding (bank spread)

template <int T, int NCOLS, int R>
__host__ __device__ constexpr int warp_smem_bytes(int stages) {
  // stage ring + parked block values (32-wide formats) + per-stage (task, chunk) words, 16-byte rounded
  return stages * R * Geo<T>::CB + (is_k_type(T) ? 0 : R * NCOLS * CHAIN_ROW * 4) + ((2 * stages * 4 + 15) / 16) * 16;
}

template <int T, int NCOLS, int R, int STAGES, int WARPS, bool ARGMAX>
__global__ void __launch_bounds__(WARPS * 32)
gemv_stream_kernel(const GemvArgs p) {
  constexpr int CB = Geo<T>::CB;
  constexpr int V = CB / 16;  // 16-byte vectors per row chunk
  constexpr bool KQ = is_k_type(T);
  static_assert(KQ || R * NCOLS <= 32, "one lane per (row, column) walks the block values");
  extern __shared__ __align__(16) uint8_t smem[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  uint8_t* ring = smem + (size_t)warp * warp_smem_bytes<T, NCOLS, R>(STAGES);
  float* chain = reinterpret_cast<float*>(ring + STAGES * R * CB);

  const int nchunks = p.K / CHUNK;
  const int ntasks = (p.M + R - 1) / R;
  // Tasks (R rows each) are handed out through an atomic counter, so a warp that
  // finishes early takes more and the launch has no long tail.  Per stage the warp
  // records which (task, chunk) the stage holds; task -1 marks the end.
  int* meta = reinterpret_cast<int*>(ring + warp_smem_bytes<T, NCOLS, R>(STAGES)) - 2 * STAGES;
  int iss_task = 0, iss_chunk = nchunks;
  bool drained = false;
  auto issue_next = [&](int slot) {
    if (iss_chunk == nchunks && !drained) {
      int t = 0;
      if (lane == 0) t = atomicAdd(p.sched, 1);
      iss_task = __shfl_sync(0xffffffffu, t, 0);
      iss_chunk = 0;
      drained = iss_task >= ntasks;
    }
    if (!drained) {
      const int row0 = iss_task * R;
      uint8_t* dst = ring + (size_t)slot * R * CB;
      for (int i = lane; i < R * V; i += 32) {
        const int r = i / V, o = i - r * V;
        const int row = min(row0 + r, p.M - 1);
        cp_async16(dst + r * CB + o * 16, p.W + (size_t)row * p.row_bytes + (size_t)iss_chunk * CB + (size_t)o * 16);
      }
    }
    if (lane == 0) {
      meta[2 * slot] = drained ? -1 : iss_task;
      meta[2 * slot + 1] = iss_chunk;
    }
    if (!drained) ++iss_chunk;
  };

#pragma unroll
  for (int s = 0; s < STAGES - 1; ++s) {
    issue_next(s);
    cp_async_commit();
  }

  // K-quants: every lane carries all R*NCOLS row sums (they stay identical across
  // lanes); 32-wide formats: lane (r*NCOLS + j) carries the sum of (row r, column j)
  float acc[KQ ? R : 1][KQ ? NCOLS : 1];
  float best = -INFINITY;
  int best_i = 0x7fffffff;

  int slot_c = 0, slot_i = STAGES - 1;
  for (;;) {
    issue_next(slot_i);
    cp_async_commit();
    slot_i = slot_i + 1 == STAGES ? 0 : slot_i + 1;
    cp_async_wait<STAGES - 1>();
    __syncwarp();

    const int task = meta[2 * slot_c], c = meta[2 * slot_c + 1];
    if (task < 0) break;
    if (c == 0) {
#pragma unroll
      for (int r = 0; r < (KQ ? R : 1); ++r)
#pragma unroll
        for (int j = 0; j < (KQ ? NCOLS : 1); ++j) acc[r][j] = 0.0f;
    }
    const uint8_t* st = ring + (size_t)slot_c * R * CB;

    auto consume = [&](int r, int j, const WRegs<T>& w, const ARegs<T>& a) {
      if constexpr (KQ) {
        const float bv = w.block_value(a);
        float s = acc[r][j];
#pragma unroll
        for (int b = 0; b < 8; ++b) s = __fadd_rn(s, __shfl_sync(0xffffffffu, bv, 4 * b));
        acc[r][j] = s;
      } else {
        const float2 bv = w.block_values(a);
        *reinterpret_cast<float2*>(chain + (r * NCOLS + j) * CHAIN_ROW + 2 * lane) = bv;
      }
    };

    if constexpr (NCOLS == 1) {
      ARegs<T> a;
      a.load(p.act, p.col0, c, lane);
#pragma unroll
      for (int r = 0; r < R; ++r) {
        WRegs<T> w;
        w.load(st + r * CB, lane);
        consume(r, 0, w, a);
      }
    } else {
#pragma unroll
      for (int r = 0; r < R; ++r) {
        WRegs<T> w;
        w.load(st + r * CB, lane);
#pragma unroll
        for (int j = 0; j < NCOLS; ++j) {
          ARegs<T> a;
          a.load(p.act, p.col0 + j, c, lane);
          consume(r, j, w, a);
        }
      }
    }
    __syncwarp();  // stage fully read (and, for the 32-wide formats, block values parked)
    if constexpr (!KQ) {
      if (lane < R * NCOLS) {
        const float4* cv = reinterpret_cast<const float4*>(chain + lane * CHAIN_ROW);
        float s = acc[0][0];
#pragma unroll
        for (int b = 0; b < 16; ++b) {
          const float4 v = cv[b];
          s = __fadd_rn(__fadd_rn(__fadd_rn(__fadd_rn(s, v.x), v.y), v.z), v.w);
        }
        acc[0][0] = s;
      }
      __syncwarp();
    }

    if (c == nchunks - 1) {
      const int row0 = task * R;
      if constexpr (KQ) {
#pragma unroll
        for (int r = 0; r < R; ++r) {
#pragma unroll
          for (int j = 0; j < NCOLS; ++j) {
            const float v = acc[r][j];
            const int row = row0 + r;
            if (row < p.M) {
              if constexpr (ARGMAX) {
                // ascending rows inside a warp; strict > keeps the lowest row on ties
                if (v > best || best_i == 0x7fffffff) { best = v; best_i = row; }
              } else if (lane == 0) {
                const size_t o = (size_t)row * p.ldy + p.col0 + j;
                p.y[o] = p.residual ? __fadd_rn(p.residual[o], v) : v;
              }
            }
          }
        }
      } else {
#pragma unroll
        for (int q = 0; q < R * NCOLS; ++q) {
          const float v = __shfl_sync(0xffffffffu, acc[0][0], q);
          const int row = row0 + q / NCOLS, j = q % NCOLS;
          if (row < p.M) {
            if constexpr (ARGMAX) {
              if (v > best || best_i == 0x7fffffff) { best = v; best_i = row; }
            } else if (lane == 0) {
              const size_t o = (size_t)row * p.ldy + p.col0 + j;
              p.y[o] = p.residual ? __fadd_rn(p.residual[o], v) : v;
            }
          }
        }
      }
    }
    slot_c = slot_c + 1 == STAGES ? 0 : slot_c + 1;
  }
  cp_async_wait<0>();
  // the last block to finish rearms the task counter for the next launch
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(p.sched + 1, 1) == (int)gridDim.x - 1) {
      p.sched[0] = 0;
      p.sched[1] = 0;
      __threadfence();
    }
  }

  if constexpr (ARGMAX) {
    __shared__ float sv[WARPS];
    __shared__ int si[WARPS];
    if (lane == 0) { sv[warp] = best; si[warp] = best_i; }
    __syncthreads();
    if (threadIdx.x == 0) {
      float bv = sv[0]; int bi = si[0];
      for (int w = 1; w < WARPS; ++w) {
        if (si[w] != 0x7fffffff && (bi == 0x7fffffff || sv[w] > bv || (sv[w] == bv && si[w] < bi))) { bv = sv[w]; bi = si[w]; }
      }
      p.part_val[blockIdx.x] = bv;
      p.part_idx[blockIdx.x] = bi;
    }
  }
}

// final reduce of per-block (value, row) candidates: maximum value, lowest row on
// ties — what a strict `>` scan over ascending rows yields
// (src/emel/kernel/detail.hpp:3720-3723)
__global__ void argmax_finish_kernel(const float* pv, const int* pi, int n, float* out_val, int* out_idx) {
  __shared__ float sv[256];
  __shared__ int si[256];
  float bv = -INFINITY; int bi = 0x7fffffff;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const float v = pv[i]; const int r = pi[i];
    if (r != 0x7fffffff && (bi == 0x7fffffff || v > bv || (v == bv && r < bi))) { bv = v; bi = r; }
  }
  sv[threadIdx.x] = bv; si[threadIdx.x] = bi;
  __syncthreads();
  for (int s = blockDim.x / 2; s > 0; s >>= 1) {
    if (threadIdx.x < s) {
      const float v = sv[threadIdx.x + s]; const int r = si[threadIdx.x + s];
      const float cv = sv[threadIdx.x]; const int cr = si[threadIdx.x];
      if (r != 0x7fffffff && (cr == 0x7fffffff || v > cv || (v == cv && r < cr))) { sv[threadIdx.x] = v; si[threadIdx.x] = r; }
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) { *out_val = sv[0]; *out_idx = si[0]; }
}

// greedy id over materialised logits: maximum value, lowest index on ties
__global__ void argmax_f32_kernel(const float* x, int n, float* out_val, int* out_idx) {
  __shared__ float sv[1024];
  __shared__ int si[1024];
  float bv = -INFINITY; int bi = 0x7fffffff;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const float v = x[i];
    if (bi == 0x7fffffff || v > bv) { bv = v; bi = i; }
  }
  sv[threadIdx.x] = bv; si[threadIdx.x] = bi;
  __syncthreads();
  for (int s = blockDim.x / 2; s > 0; s >>= 1) {
    if (threadIdx.x < s) {
      const float v = sv[threadIdx.x + s]; const int r = si[threadIdx.x + s];
      const float cv = sv[threadIdx.x]; const int cr = si[threadIdx.x];
      if (r != 0x7fffffff && (cr == 0x7fffffff || v > cv || (v == cv && r < cr))) { sv[threadIdx.x] = v; si[threadIdx.x] = r; }
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) { *out_val = sv[0]; *out_idx = si[0]; }
}

// ---------------------------------------------------------------- generic kernel
// Any K that is a multiple of the block size, any 2-byte-aligned base: one warp
// per row, lanes stride over blocks, byte loads.  Used for shapes the streaming
// kernel does not take (K % 2048 != 0 or an unaligned view); not a fast path.
__device__ __forceinline__ int scale_min_k4_sc(int j, const uint8_t* q) {
  return j < 4 ? (q[j] & 63) : ((q[j + 4] & 0x0f) | ((q[j - 4] >> 6) << 4));
}
__device__ __forceinline__ int scale_min_k4_m(int j, const uint8_t* q) {
  return j < 4 ? (q[j + 4] & 63) : ((q[j + 4] >> 4) | ((q[j] >> 6) << 4));
}
__device__ __forceinline__ uint16_t ld16(const uint8_t* p) { return (uint16_t)p[0] | ((uint16_t)p[1] << 8); }

template <int T>
__device__ float generic_block_dot(const uint8_t* blk, const ActPlanes& act, int col, int64_t ib) {
  const int8_t* a = act.qs + col * act.col_stride_qs + ib * block_elems(T);
  if constexpr (T == T_Q4_K) {
    const float d = h2f(ld16(blk)), dmin = h2f(ld16(blk + 2));
    const uint8_t* s = blk + 4;
    const uint8_t* q = blk + 16;
    const int16_t* bs = act.bsums + col * act.col_stride_bs + ib * 16;
    int isum = 0, msum = 0;
    for (int j = 0; j < 8; ++j) {
      int dot = 0;
      const uint8_t* qq = q + 32 * (j >> 1);
      for (int l = 0; l < 32; ++l) dot += (int)((j & 1) ? (qq[l] >> 4) : (qq[l] & 0x0f)) * (int)a[32 * j + l];
      isum += scale_min_k4_sc(j, s) * dot;
      msum += scale_min_k4_m(j, s) * ((int)bs[2 * j] + (int)bs[2 * j + 1]);
    }
    const float dx = act.d[col * act.col_stride_d + ib];
    return __fmaf_rn(__fmul_rn(dx, d), (float)isum, -__fmul_rn(__fmul_rn(dx, dmin), (float)msum));
  } else if constexpr (T == T_Q6_K) {
    const uint8_t* ql = blk; const uint8_t* qh = blk + 128;
    const int8_t* sc = reinterpret_cast<const int8_t*>(blk + 192);
    const float d = h2f(ld16(blk + 208));
    int isum = 0;
    for (int n = 0; n < 2; ++n) {
      for (int l = 0; l < 32; ++l) {
        const int is = l / 16;
        const int q1 = (int)((ql[64 * n + l] & 0x0f) | (((qh[32 * n + l] >> 0) & 3) << 4)) - 32;
        const int q2 = (int)((ql[64 * n + l + 32] & 0x0f) | (((qh[32 * n + l] >> 2) & 3) << 4)) - 32;
        const int q3 = (int)((ql[64 * n + l] >> 4) | (((qh[32 * n + l] >> 4) & 3) << 4)) - 32;
        const int q4 = (int)((ql[64 * n + l + 32] >> 4) | (((qh[32 * n + l] >> 6) & 3) << 4)) - 32;
        isum += (int)sc[8 * n + is + 0] * q1 * (int)a[128 * n + l];
        isum += (int)sc[8 * n + is + 2] * q2 * (int)a[128 * n + l + 32];
        isum += (int)sc[8 * n + is + 4] * q3 * (int)a[128 * n + l + 64];
        isum += (int)sc[8 * n + is + 6] * q4 * (int)a[128 * n + l + 96];
      }
    }
    return __fmul_rn(__fmul_rn(act.d[col * act.col_stride_d + ib], d), (float)isum);
  } else if constexpr (T == T_Q8_0) {
    const int8_t* q = reinterpret_cast<const int8_t*>(blk + 2);
    int s = 0;
    for (int l = 0; l < 32; ++l) s += (int)q[l] * (int)a[l];
    return __fmul_rn((float)s, __fmul_rn(h2f(ld16(blk)), act.d[col * act.col_stride_d + ib]));
  } else {
    const uint8_t* q = blk + 2;
    int s = 0;
    for (int l = 0; l < 16; ++l) {
      s += ((int)(q[l] & 0x0f) - 8) * (int)a[l];
      s += ((int)(q[l] >> 4) - 8) * (int)a[l + 16];
    }
    return __fmul_rn((float)s, __fmul_rn(h2f(ld16(blk)), act.d[col * act.col_stride_d + ib]));
  }
}

template <int T, bool ARGMAX>
__global__ void __launch_bounds__(128) gemv_generic_kernel(const GemvArgs p, int ncols) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nblk = p.K / block_elems(T);
  float best = -INFINITY; int best_i = 0x7fffffff;
  for (int row = blockIdx.x * 4 + warp; row < p.M; row += gridDim.x * 4) {
    const uint8_t* wrow = p.W + (size_t)row * p.row_bytes;
    for (int j = 0; j < ncols; ++j) {
      float acc = 0.0f;
      // 32 block values at a time, added in ascending block order
      for (int base = 0; base < nblk; base += 32) {
        const int ib = base + lane;
        const float bv = ib < nblk ? generic_block_dot<T>(wrow + (size_t)ib * block_bytes(T), p.act, p.col0 + j, ib) : 0.0f;
        const int cnt = min(32, nblk - base);
        for (int i = 0; i < cnt; ++i) acc = __fadd_rn(acc, __shfl_sync(0xffffffffu, bv, i));
      }
      if constexpr (ARGMAX) {
        if (acc > best || best_i == 0x7fffffff) { best = acc; best_i = row; }
      } else if (lane == 0) {
        const size_t o = (size_t)row * p.ldy + p.col0 + j;
        p.y[o] = p.residual ? __fadd_rn(p.residual[o], acc) : acc;
      }
    }
  }
  if constexpr (ARGMAX) {
    __shared__ float sv[4];
    __shared__ int si[4];
    if (lane == 0) { sv[warp] = best; si[warp] = best_i; }
    __syncthreads();
    if (threadIdx.x == 0) {
      float bv = sv[0]; int bi = si[0];
      for (int w = 1; w < 4; ++w)
        if (si[w] != 0x7fffffff && (bi == 0x7fffffff || sv[w] > bv || (sv[w] == bv && si[w] < bi))) { bv = sv[w]; bi = si[w]; }
      p.part_val[blockIdx.x] = bv;
      p.part_idx[blockIdx.x] = bi;
    }
  }
}

// ---------------------------------------------------------------- launch logic
constexpr int kWarps = 4;
constexpr int kStages = 3;

template <int T, int NCOLS, int R, bool ARGMAX>
cudaError_t launch_stream(const GemvArgs& a, int sm_count, cudaStream_t st, int* grid_out) {
  constexpr size_t smem = (size_t)kWarps * warp_smem_bytes<T, NCOLS, R>(kStages);
  auto kern = gemv_stream_kernel<T, NCOLS, R, kStages, kWarps, ARGMAX>;
  static unsigned configured = 0;  // per instantiation, one bit per device
  int dev = 0;
  cudaGetDevice(&dev);
  if (!(configured & (1u << (dev & 31)))) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    configured |= 1u << (dev & 31);
  }
  const int ntasks = (a.M + R - 1) / R;
  const int per_sm = (int)((220 * 1024) / smem) > 0 ? (int)((220 * 1024) / smem) : 1;
  int grid = (ntasks + kWarps - 1) / kWarps;
  const int cap = sm_count * (per_sm > 8 ? 8 : per_sm);
  if (grid > cap) grid = cap;
  if (ARGMAX && grid > kMaxArgmaxParts) grid = kMaxArgmaxParts;
  if (grid_out) *grid_out = grid;
  kern<<<grid, kWarps * 32, smem, st>>>(a);
  return cudaGetLastError();
}

// rows per task: more rows share one activation register set, fewer rows give
// finer scheduling granules and more resident warps.  EMELB_GEMV_R overrides.
inline int rows_per_task_override() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("EMELB_GEMV_R");
    v = e ? atoi(e) : 0;
  }
  return v;
}

template <int T, int NCOLS, bool ARGMAX>
cudaError_t launch_pick_r(const GemvArgs& a, int sm_count, cudaStream_t st, int* grid_out) {
  int r = a.M >= sm_count * kWarps * 4 ? 2 : 1;
  if (rows_per_task_override() > 0) r = rows_per_task_override();
  if constexpr (NCOLS == 1) {
    if (r >= 4) return launch_stream<T, NCOLS, 4, ARGMAX>(a, sm_count, st, grid_out);
    if (r >= 2) return launch_stream<T, NCOLS, 2, ARGMAX>(a, sm_count, st, grid_out);
    return launch_stream<T, NCOLS, 1, ARGMAX>(a, sm_count, st, grid_out);
  } else {
    if (r >= 2) return launch_stream<T, NCOLS, 2, ARGMAX>(a, sm_count, st, grid_out);
    return launch_stream<T, NCOLS, 1, ARGMAX>(a, sm_count, st, grid_out);
  }
}

template <int T>
cudaError_t launch_type(GemvArgs a, int ncols, bool argmax, bool fast, int sm_count, cudaStream_t st, int* launches,
                        int* grid_out) {
  cudaError_t e = cudaSuccess;
  if (!fast) {
    int grid = (a.M + 3) / 4;
    if (grid > sm_count * 8) grid = sm_count * 8;
    if (argmax && grid > kMaxArgmaxParts) grid = kMaxArgmaxParts;
    if (grid_out) *grid_out = grid;
    if (argmax) gemv_generic_kernel<T, true><<<grid, 128, 0, st>>>(a, 1);
    else gemv_generic_kernel<T, false><<<grid, 128, 0, st>>>(a, ncols);
    ++*launches;
    return cudaGetLastError();
  }
  // second-generation streaming kernel (gemv2.cu) unless EMELB_GEMV_V1 asks for the first
  static const bool v1 = getenv("EMELB_GEMV_V1") != nullptr;
  if (!v1) return launch_gemv_stream2(T, a, ncols, argmax, sm_count, st, launches, grid_out);
  if (argmax) {
    ++*launches;
    return launch_pick_r<T, 1, true>(a, sm_count, st, grid_out);
  }
  int done = 0;
  while (done < ncols && e == cudaSuccess) {
    GemvArgs b = a;
    b.col0 = a.col0 + done;
    const int left = ncols - done;
    if (left >= 8) { e = launch_pick_r<T, 8, false>(b, sm_count, st, grid_out); done += 8; }
    else if (left >= 4) { e = launch_pick_r<T, 4, false>(b, sm_count, st, grid_out); done += 4; }
    else if (left >= 2) { e = launch_pick_r<T, 2, false>(b, sm_count, st, grid_out); done += 2; }
    else { e = launch_pick_r<T, 1, false>(b, sm_count, st, grid_out); done += 1; }
    ++*launches;
  }
  return e;
}

}  // namespace

cudaError_t launch_argmax_f32(const float* x, int n, float* out_val, int* out_idx, cudaStream_t st) {
  argmax_f32_kernel<<<1, 1024, 0, st>>>(x, n, out_val, out_idx);
  return cudaGetLastError();
}

bool gemv_fast_path_ok(int type, const void* w, int64_t row_bytes, int K) {
  (void)type;
  return (K % CHUNK) == 0 && (reinterpret_cast<uintptr_t>(w) % 16) == 0 && (row_bytes % 16) == 0;
}

bool gemv_takes_tensor_core(int type, const GemvArgs& a, int ncols) {
  static const bool no_tc = getenv("EMELB_NO_TC") != nullptr;
  return !no_tc && a.tc_ws && gemm_tc_supported(type, a.K, ncols, a.W, a.row_bytes, a.act) &&
         gemm_tc_workspace_bytes(a.K, ncols) <= a.tc_ws_bytes;
}

cudaError_t launch_gemv(int type, const GemvArgs& a, int ncols, bool argmax, int sm_count, cudaStream_t st,
                        int* launches) {
  // many columns of Q8_0 / Q4_0: one tensor-core instruction per 32-weight block (gemm_q8_mma.cu)
  if (!argmax && gemm_q8_mma_supported(type, a, ncols)) {
    ++*launches;
    return launch_gemm_q8_mma(type, a, ncols, sm_count, st);
  }
  // many columns of Q4_K: the tensor-core kernel (same numbers, see gemm_tc.cu)
  if (!argmax && gemv_takes_tensor_core(type, a, ncols)) {
    *launches += a.tc_ws_reuse ? 1 : 2;
    return launch_gemm_q4k_tc(a, ncols, sm_count, a.tc_ws, st);
  }
  const bool fast = gemv_fast_path_ok(type, a.W, a.row_bytes, a.K);
  int grid = 0;
  cudaError_t e;
  switch (type) {
    case T_Q4_K: e = launch_type<T_Q4_K>(a, ncols, argmax, fast, sm_count, st, launches, &grid); break;
    case T_Q6_K: e = launch_type<T_Q6_K>(a, ncols, argmax, fast, sm_count, st, launches, &grid); break;
    case T_Q8_0: e = launch_type<T_Q8_0>(a, ncols, argmax, fast, sm_count, st, launches, &grid); break;
    case T_Q4_0: e = launch_type<T_Q4_0>(a, ncols, argmax, fast, sm_count, st, launches, &grid); break;
    default: return cudaErrorInvalidValue;
  }
  if (e != cudaSuccess) return e;
  if (argmax) {
    argmax_finish_kernel<<<1, 256, 0, st>>>(a.part_val, a.part_idx, grid, a.best_val, a.best_idx);
    ++*launches;
    e = cudaGetLastError();
  }
  return e;
}

}  // namespace emelb
