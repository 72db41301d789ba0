// Streaming mat-vec, second generation: one lane per 256 weights.
//
// Same contract and same float order as gemv.cu's first streaming kernel (the
// reference's x86 route block by block, see the notes there); what changes is
// how a warp spends its instructions, because that kernel turned out to be
// bound by instruction issue (about 270 warp instructions per 2048-weight row
// chunk, 46 % issue utilisation at 20 % of HBM bandwidth), not by memory:
//   * copies: one elected lane issues one bulk-async copy (TMA unit,
//     cp.async.bulk) per row chunk into the warp's private stage ring and the
//     warp waits on an mbarrier — no per-lane copy instructions or address math;
//   * a stage holds 4 rows x 2048 weights, i.e. 32 spans of 256 weights: lane
//     (r, b) = (lane / 8, lane % 8) owns span b of row r, so the 6-bit scale
//     unpacking, the integer reductions and the block value need no shuffles,
//     and the block-order row sum costs 8 shuffles + 8 adds per 4 rows;
//   * the 256 activations a lane needs depend only on b: they are loaded once per
//     chunk into registers and reused for every 4-row pass of the task.
// Every mbarrier wait is bounded; a wait that runs out raises the status word
// the host turns into internal_error, and the warp leaves.
#include <cstdlib>

#include "common.cuh"
#include "kernels.h"
#include "peer_join.cuh"
#include "quant_device.cuh"

namespace emelb {

namespace {

constexpr int CHUNK = 2048;
constexpr int ROWS_PER_STAGE = 4;

template <int T> struct Geo2;
template <> struct Geo2<T_Q4_K> { static constexpr int CB = 8 * Q4_K_BYTES; };
template <> struct Geo2<T_Q6_K> { static constexpr int CB = 8 * Q6_K_BYTES; };
template <> struct Geo2<T_Q8_0> { static constexpr int CB = 64 * Q8_0_BYTES; };
template <> struct Geo2<T_Q4_0> { static constexpr int CB = 64 * Q4_0_BYTES; };

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// global -> this CTA's shared memory, completion counted in bytes on `bar`;
// both addresses 16-byte aligned, size a multiple of 16
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(dst)),
               "l"(src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

__device__ __forceinline__ int dp4a_us(uint32_t a_unsigned, int b_signed, int c) {
  int d;
  asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a_unsigned), "r"(b_signed), "r"(c));
  return d;
}

// ---------------------------------------------------------------- activations
// the 256 quantized activations of span b of chunk c, one column
struct Act256 {
  int a[64];
  int bs[8];   // Q8_K: sums of the 8 sub-blocks of 32 (pairs of 16-wide bsums); unused for Q8_0
  int bs16[16];
  float d[8];  // Q8_K: d[0]; Q8_0: the 8 block scales
};

template <bool KQ, bool NEED16>
__device__ __forceinline__ void load_act(Act256& x, const ActPlanes& act, int col, int chunk, int b) {
  const int64_t e0 = (int64_t)chunk * CHUNK + 256 * b;
  const int4* q = reinterpret_cast<const int4*>(act.qs + col * act.col_stride_qs + e0);
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const int4 v = __ldg(q + i);
    x.a[4 * i + 0] = v.x; x.a[4 * i + 1] = v.y; x.a[4 * i + 2] = v.z; x.a[4 * i + 3] = v.w;
  }
  if constexpr (KQ) {
    const int4* s = reinterpret_cast<const int4*>(act.bsums + col * act.col_stride_bs + e0 / 16);
    const int4 s0 = __ldg(s), s1 = __ldg(s + 1);
    const int w[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int lo = (int)(short)(w[j] & 0xffff), hi = w[j] >> 16;
      x.bs[j] = lo + hi;
      if constexpr (NEED16) { x.bs16[2 * j] = lo; x.bs16[2 * j + 1] = hi; }
    }
    x.d[0] = __ldg(act.d + col * act.col_stride_d + e0 / QK_K);
  } else {
    const float4* dd = reinterpret_cast<const float4*>(act.d + col * act.col_stride_d + e0 / 32);
    const float4 d0 = __ldg(dd), d1 = __ldg(dd + 1);
    x.d[0] = d0.x; x.d[1] = d0.y; x.d[2] = d0.z; x.d[3] = d0.w;
    x.d[4] = d1.x; x.d[5] = d1.y; x.d[6] = d1.z; x.d[7] = d1.w;
  }
}

// ---------------------------------------------------------------- block values
// Q4_K super-block at a 16-byte aligned shared address: value of the block
// against the lane's activations, fma(d*dx, isum, -(dmin*dx)*msum)
// (src/emel/kernel/x86_64/actions.hpp:859-866); scales/mins per
// get_scale_min_k4 through the kmask word shuffle (:793-801)
__device__ __forceinline__ float q4_k_block_value(const uint8_t* blk, const Act256& x) {
  const uint4 h = *reinterpret_cast<const uint4*>(blk);
  const uint32_t s0 = h.y, s1 = h.z, s2 = h.w;
  const uint32_t sc_lo = s0 & 0x3f3f3f3fu;                                        // scales 0..3
  const uint32_t mn_lo = s1 & 0x3f3f3f3fu;                                        // mins 0..3
  const uint32_t sc_hi = (s2 & 0x0f0f0f0fu) | (((s0 >> 6) & 0x03030303u) << 4);   // scales 4..7
  const uint32_t mn_hi = ((s2 >> 4) & 0x0f0f0f0fu) | (((s1 >> 6) & 0x03030303u) << 4);
  int isum = 0, msum = 0;
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    const uint4 v0 = *reinterpret_cast<const uint4*>(blk + 16 + 32 * r);
    const uint4 v1 = *reinterpret_cast<const uint4*>(blk + 32 + 32 * r);
    const uint32_t q[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
    int lo = 0, hi16 = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      lo = __dp4a((int)(q[i] & 0x0f0f0f0fu), x.a[16 * r + i], lo);
      hi16 = dp4a_us(q[i] & 0xf0f0f0f0u, x.a[16 * r + 8 + i], hi16);   // 16 x the high-nibble dot
    }
    const uint32_t scw = r < 2 ? sc_lo : sc_hi, mnw = r < 2 ? mn_lo : mn_hi;
    const int sh = 16 * (r & 1);
    isum += (int)((scw >> sh) & 0xff) * lo + (int)((scw >> (sh + 8)) & 0xff) * (hi16 >> 4);
    msum += (int)((mnw >> sh) & 0xff) * x.bs[2 * r] + (int)((mnw >> (sh + 8)) & 0xff) * x.bs[2 * r + 1];
  }
  const float d = h2f((uint16_t)(h.x & 0xffffu)), dmin = h2f((uint16_t)(h.x >> 16));
  const float d_all = __fmul_rn(x.d[0], d), d_min = __fmul_rn(x.d[0], dmin);
  return __fmaf_rn(d_all, (float)isum, -__fmul_rn(d_min, (float)msum));
}

// Q6_K super-block at a 2-byte aligned shared address (210-byte blocks): the 52
// payload words are realigned with funnel shifts, then
// (dx*d) * sum_g scale_g * (dot16_g - 32*bsum_g)
// (src/emel/kernel/x86_64/actions.hpp:1036-1077; layout src/emel/kernel/detail.hpp:592-629)
__device__ __forceinline__ float q6_k_block_value(const uint8_t* blk, const Act256& x) {
  const uint32_t addr = smem_u32(blk);
  const uint32_t base = addr & ~3u;
  const int sh = (addr & 2u) * 8;
  uint32_t w[53];
#pragma unroll
  for (int i = 0; i < 53; ++i) asm volatile("ld.shared.u32 %0, [%1];" : "=r"(w[i]) : "r"(base + 4 * i));
  uint32_t u[52];  // ql: u[0..31], qh: u[32..47], scales: u[48..51]
#pragma unroll
  for (int i = 0; i < 52; ++i) u[i] = __funnelshift_r(w[i], w[i + 1], sh);
  const uint32_t dbits = sh ? (w[52] >> 16) : (w[52] & 0xffffu);
  int isum = 0;
#pragma unroll
  for (int n = 0; n < 2; ++n) {
    int s[8];
#pragma unroll
    for (int g = 0; g < 8; ++g) s[g] = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const uint32_t qa = u[16 * n + i], qb = u[16 * n + 8 + i], qh = u[32 + 8 * n + i];
      const uint32_t v1 = (qa & 0x0f0f0f0fu) | ((qh & 0x03030303u) << 4);
      const uint32_t v2 = (qb & 0x0f0f0f0fu) | (((qh >> 2) & 0x03030303u) << 4);
      const uint32_t v3 = ((qa >> 4) & 0x0f0f0f0fu) | (((qh >> 4) & 0x03030303u) << 4);
      const uint32_t v4 = ((qb >> 4) & 0x0f0f0f0fu) | (((qh >> 6) & 0x03030303u) << 4);
      const int g = i >> 2;  // which 16-wide group inside each 32-wide quarter
      s[0 + g] = __dp4a((int)v1, x.a[32 * n + i], s[0 + g]);
      s[2 + g] = __dp4a((int)v2, x.a[32 * n + 8 + i], s[2 + g]);
      s[4 + g] = __dp4a((int)v3, x.a[32 * n + 16 + i], s[4 + g]);
      s[6 + g] = __dp4a((int)v4, x.a[32 * n + 24 + i], s[6 + g]);
    }
#pragma unroll
    for (int g = 0; g < 8; ++g) {
      const int sc = (int)(int8_t)((u[48 + 2 * n + (g >> 2)] >> (8 * (g & 3))) & 0xff);
      isum += sc * (s[g] - 32 * x.bs16[8 * n + g]);
    }
  }
  return __fmul_rn(__fmul_rn(x.d[0], h2f((uint16_t)dbits)), (float)isum);
}

// eight consecutive Q8_0 blocks = 272 bytes at a 16-byte aligned shared address;
// per block (float)sumi * (h(dw) * h(dx)) (src/emel/kernel/detail.hpp:3257-3266)
__device__ __forceinline__ void q8_0_block_values(const uint8_t* span, const Act256& x, float (&bv)[8]) {
  uint32_t w[68];
#pragma unroll
  for (int i = 0; i < 17; ++i) {
    const uint4 v = *reinterpret_cast<const uint4*>(span + 16 * i);
    w[4 * i] = v.x; w[4 * i + 1] = v.y; w[4 * i + 2] = v.z; w[4 * i + 3] = v.w;
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int w0 = 17 * (j >> 1) + ((j & 1) ? 8 : 0);
    int s = 0;
    float dw;
    if ((j & 1) == 0) {
      dw = h2f((uint16_t)(w[w0] & 0xffffu));
#pragma unroll
      for (int i = 0; i < 8; ++i) s = __dp4a((int)__funnelshift_r(w[w0 + i], w[w0 + i + 1], 16), x.a[8 * j + i], s);
    } else {
      dw = h2f((uint16_t)(w[w0] >> 16));
#pragma unroll
      for (int i = 0; i < 8; ++i) s = __dp4a((int)w[w0 + 1 + i], x.a[8 * j + i], s);
    }
    bv[j] = __fmul_rn((float)s, __fmul_rn(dw, x.d[j]));
  }
}

// eight consecutive Q4_0 blocks = 144 bytes; element l = low nibble of byte l,
// element l+16 = high nibble, value = nibble - 8 (src/emel/kernel/detail.hpp:3131-3153)
__device__ __forceinline__ void q4_0_block_values(const uint8_t* span, const Act256& x, float (&bv)[8]) {
  uint32_t w[36];
#pragma unroll
  for (int i = 0; i < 9; ++i) {
    const uint4 v = *reinterpret_cast<const uint4*>(span + 16 * i);
    w[4 * i] = v.x; w[4 * i + 1] = v.y; w[4 * i + 2] = v.z; w[4 * i + 3] = v.w;
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int w0 = 9 * (j >> 1) + ((j & 1) ? 4 : 0);
    int s = 0, t = 0;
    float dw;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      uint32_t q;
      if ((j & 1) == 0) q = __funnelshift_r(w[w0 + i], w[w0 + i + 1], 16);
      else q = w[w0 + 1 + i];
      s = __dp4a((int)(q & 0x0f0f0f0fu), x.a[8 * j + i], s);
      s = __dp4a((int)((q >> 4) & 0x0f0f0f0fu), x.a[8 * j + 4 + i], s);
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) t = __dp4a(0x01010101, x.a[8 * j + i], t);
    dw = (j & 1) == 0 ? h2f((uint16_t)(w[w0] & 0xffffu)) : h2f((uint16_t)(w[w0] >> 16));
    bv[j] = __fmul_rn((float)(s - 8 * t), __fmul_rn(dw, x.d[j]));
  }
}

// ---------------------------------------------------------------- kernel
template <int T, int STAGES>
__host__ __device__ constexpr int warp_bytes2() {
  // stage ring + STAGES mbarriers + STAGES (task, chunk, pass) records, 16-byte rounded
  return STAGES * ROWS_PER_STAGE * Geo2<T>::CB + ((STAGES * 8 + STAGES * 16 + 15) / 16) * 16;
}

constexpr int kWaitLimit = 1 << 22;
constexpr unsigned long long kWaitLimitNs = 1000000000ull;  // 1 s

// One task = 4*RP rows (RP passes of 4 rows); its items run chunk-major, pass-minor,
// so a row meets its chunks in ascending order and the activations of a chunk serve
// all passes.
template <int T, int NCOLS, int RP, int STAGES, int WARPS, bool ARGMAX>
__global__ void __launch_bounds__(WARPS * 32)
gemv2_kernel(const GemvArgs p) {
  constexpr int CB = Geo2<T>::CB;
  constexpr bool KQ = is_k_type(T);
  constexpr int SPAN = CB / 8;  // bytes of 256 weights of one row
  extern __shared__ __align__(128) uint8_t smem2[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  uint8_t* ring = smem2 + (size_t)warp * warp_bytes2<T, STAGES>();
  uint64_t* bars = reinterpret_cast<uint64_t*>(ring + STAGES * ROWS_PER_STAGE * CB);
  int* meta = reinterpret_cast<int*>(bars + STAGES);  // 4 ints per stage: task, chunk, pass, -

  const int nchunks = p.K / CHUNK;
  const int rows_per_task = ROWS_PER_STAGE * RP;
  // tasks of the (up to three) matrices are numbered back to back
  const int nt0 = (p.M + rows_per_task - 1) / rows_per_task;
  const int nt1 = (p.M2 + rows_per_task - 1) / rows_per_task;
  const int nt2 = (p.M3 + rows_per_task - 1) / rows_per_task;
  const int ntasks = nt0 + nt1 + nt2;

  if (lane == 0) {
#pragma unroll
    for (int s = 0; s < STAGES; ++s) mbar_init(bars + s, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  __syncwarp();

  // the first task of a warp is its global index; later ones come from the counter
  const int total_warps = gridDim.x * WARPS;
  int iss_task = blockIdx.x * WARPS + warp, iss_chunk = 0, iss_pass = 0;
  bool drained = iss_task >= ntasks;
  pdl_trigger();
  auto issue_next = [&](int slot) {
    if (!drained) {
      if (iss_chunk == nchunks) {  // previous task finished: take the next one
        int t = 0;
        if (lane == 0) t = atomicAdd(p.sched, 1);
        iss_task = __shfl_sync(0xffffffffu, t, 0) + total_warps;
        iss_chunk = 0;
        iss_pass = 0;
        drained = iss_task >= ntasks;
      }
    }
    if (lane == 0) {
      meta[4 * slot] = drained ? -1 : iss_task;
      meta[4 * slot + 1] = iss_chunk;
      meta[4 * slot + 2] = iss_pass;
      if (!drained) {
        uint8_t* dst = ring + (size_t)slot * ROWS_PER_STAGE * CB;
        mbar_expect_tx(bars + slot, ROWS_PER_STAGE * CB);
        const int seg = iss_task < nt0 ? 0 : (iss_task < nt0 + nt1 ? 1 : 2);
        const int lt = iss_task - (seg == 0 ? 0 : (seg == 1 ? nt0 : nt0 + nt1));
        const uint8_t* wbase = seg == 0 ? p.W : (seg == 1 ? p.W2 : p.W3);
        const int mseg = seg == 0 ? p.M : (seg == 1 ? p.M2 : p.M3);
        const int row0 = lt * rows_per_task + iss_pass * ROWS_PER_STAGE;
#pragma unroll
        for (int r = 0; r < ROWS_PER_STAGE; ++r) {
          const int row = min(row0 + r, mseg - 1);
          bulk_g2s(dst + r * CB, wbase + (size_t)row * p.row_bytes + (size_t)iss_chunk * CB, CB, bars + slot);
        }
      }
    }
    if (!drained) {
      if (++iss_pass == RP) { iss_pass = 0; ++iss_chunk; }
    }
  };

#pragma unroll
  for (int s = 0; s < STAGES - 1; ++s) issue_next(s);
  // weights do not depend on the previous kernel; everything read below does
  pdl_wait();

  const int r4 = lane >> 3, b = lane & 7;
  float acc[RP][NCOLS];
  float best = -INFINITY;
  int best_i = 0x7fffffff;
  uint32_t phase = 0;
  int slot_c = 0, slot_i = STAGES - 1;
  bool failed = false;
  Act256 x;
  int x_task = -1, x_chunk = -1;

  for (;;) {
    issue_next(slot_i);
    slot_i = slot_i + 1 == STAGES ? 0 : slot_i + 1;
    __syncwarp();
    const int task = meta[4 * slot_c], c = meta[4 * slot_c + 1], pass = meta[4 * slot_c + 2];
    if (task < 0) break;
    if (NCOLS == 1 && (x_task != task || x_chunk != c)) {  // issued ahead of the wait: independent of the weights
      load_act<KQ, T == T_Q6_K>(x, p.act, p.col0, c, b);
      x_task = task;
      x_chunk = c;
    }
    {
      // bounded twice: by poll count and by wall time (a poll may itself block for a while)
      int spins = 0;
      bool ok = false;
      unsigned long long t_start = 0;
      while (!(ok = mbar_try_wait(bars + slot_c, (phase >> slot_c) & 1u)) && ++spins < kWaitLimit) {
        if ((spins & 255) == 0) {
          unsigned long long now;
          asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
          if (t_start == 0) t_start = now;
          else if (now - t_start > kWaitLimitNs) break;
        }
      }
      if (!__all_sync(0xffffffffu, ok)) { failed = true; break; }
      phase ^= 1u << slot_c;
    }
    if (c == 0) {
#pragma unroll
      for (int j = 0; j < NCOLS; ++j) {
#pragma unroll
        for (int q = 0; q < RP; ++q)
          if (q == pass) acc[q][j] = 0.0f;
      }
    }
    const uint8_t* st = ring + (size_t)slot_c * ROWS_PER_STAGE * CB + r4 * CB;
#pragma unroll
    for (int j = 0; j < NCOLS; ++j) {
      if (NCOLS > 1 || x_task != task || x_chunk != c) {
        load_act<KQ, T == T_Q6_K>(x, p.act, p.col0 + j, c, b);
        x_task = task;
        x_chunk = c;
      }
      float s = 0.0f;
#pragma unroll
      for (int q = 0; q < RP; ++q)
        if (q == pass) s = acc[q][j];
      if constexpr (KQ) {
        float bv;
        if constexpr (T == T_Q4_K) bv = q4_k_block_value(st + b * SPAN, x);
        else bv = q6_k_block_value(st + b * SPAN, x);
#pragma unroll
        for (int i = 0; i < 8; ++i) s = __fadd_rn(s, __shfl_sync(0xffffffffu, bv, (lane & ~7) + i));
      } else {
        float bv[8];
        if constexpr (T == T_Q8_0) q8_0_block_values(st + b * SPAN, x, bv);
        else q4_0_block_values(st + b * SPAN, x, bv);
#pragma unroll
        for (int g = 0; g < 8; ++g)
#pragma unroll
          for (int i = 0; i < 8; ++i) s = __fadd_rn(s, __shfl_sync(0xffffffffu, bv[i], (lane & ~7) + g));
      }
#pragma unroll
      for (int q = 0; q < RP; ++q)
        if (q == pass) acc[q][j] = s;
      if (c == nchunks - 1) {
        const int seg = task < nt0 ? 0 : (task < nt0 + nt1 ? 1 : 2);
        const int lt = task - (seg == 0 ? 0 : (seg == 1 ? nt0 : nt0 + nt1));
        const int mseg = seg == 0 ? p.M : (seg == 1 ? p.M2 : p.M3);
        float* yseg = seg == 0 ? p.y : (seg == 1 ? p.y2 : p.y3);
        const int row = lt * rows_per_task + pass * ROWS_PER_STAGE + r4;
        if (row < mseg) {
          if constexpr (ARGMAX) {
            if (s > best || best_i == 0x7fffffff) { best = s; best_i = row; }
          } else if (b == 0) {
            const size_t o = (size_t)row * p.ldy + p.col0 + j;
            yseg[o] = (p.residual && seg == 0) ? __fadd_rn(p.residual[o], s) : s;
          }
        }
      }
    }
    __syncwarp();  // the stage is free for the next bulk copy
    slot_c = slot_c + 1 == STAGES ? 0 : slot_c + 1;
  }
  if (failed && lane == 0 && p.status) atomicExch(p.status, 1);

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
    // lanes of a warp hold different rows: lowest row among the maxima wins
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
      if (oi != 0x7fffffff && (best_i == 0x7fffffff || ov > best || (ov == best && oi < best_i))) { best = ov; best_i = oi; }
    }
    __shared__ float sv[WARPS];
    __shared__ int si[WARPS];
    if (lane == 0) { sv[warp] = best; si[warp] = best_i; }
    __syncthreads();
    if (threadIdx.x == 0) {
      float bvv = sv[0]; int bi = si[0];
      for (int w = 1; w < WARPS; ++w)
        if (si[w] != 0x7fffffff && (bi == 0x7fffffff || sv[w] > bvv || (sv[w] == bvv && si[w] < bi))) { bvv = sv[w]; bi = si[w]; }
      p.part_val[blockIdx.x] = bvv;
      p.part_idx[blockIdx.x] = bi;
    }
  }
}

// ---------------------------------------------------------------- third generation (one column)
// Profiling the kernel above showed a warp retiring one instruction every ~13
// cycles with only 3 warps per scheduler resident (122 registers, 18 KB of stages
// per warp): the copies were fine (the same ring without arithmetic reaches the
// copy roofline), the arithmetic was latency-bound.  This variant trades software
// pipelining for thread-level parallelism: activations are staged once per CTA in
// shared memory instead of living in 70 registers per lane, each warp keeps a
// single (or two) 4-row stage(s), and up to 32 warps per SM overlap one another's
// copy latency and dependent-instruction latency.
// The eight lanes of a row read the same 16-byte unit index of eight different
// 256-byte spans at once; stored plainly those are one bank group (an 8-way
// conflict per load).  Unit i of span s is therefore kept at i ^ (s & 7).
__device__ __forceinline__ int act_swizzle(int e0) { return (e0 >> 8) & 7; }

struct ActSmem {
  const int8_t* qs;     // K int8, 16-byte units swizzled inside each 256-byte span
  const int16_t* bs;    // K/16 int16 (Q8_K only)
  const float* d;       // K/256 (Q8_K) or K/32 (Q8_0) f32
};

__device__ __forceinline__ float q4_k_block_value_s(const uint8_t* blk, const ActSmem& x, int e0) {
  const uint4 h = *reinterpret_cast<const uint4*>(blk);
  const uint32_t s0 = h.y, s1 = h.z, s2 = h.w;
  const uint32_t sc_lo = s0 & 0x3f3f3f3fu, mn_lo = s1 & 0x3f3f3f3fu;
  const uint32_t sc_hi = (s2 & 0x0f0f0f0fu) | (((s0 >> 6) & 0x03030303u) << 4);
  const uint32_t mn_hi = ((s2 >> 4) & 0x0f0f0f0fu) | (((s1 >> 6) & 0x03030303u) << 4);
  const int4* aq = reinterpret_cast<const int4*>(x.qs + e0);
  const int sw = act_swizzle(e0);
  const int4* bq = reinterpret_cast<const int4*>(x.bs + e0 / 16);
  const int4 b0 = bq[0], b1 = bq[1];
  const int bw[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
  int isum = 0, msum = 0;
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    const uint4 v0 = *reinterpret_cast<const uint4*>(blk + 16 + 32 * r);
    const uint4 v1 = *reinterpret_cast<const uint4*>(blk + 32 + 32 * r);
    const int4 a0 = aq[(4 * r) ^ sw], a1 = aq[(4 * r + 1) ^ sw], a2 = aq[(4 * r + 2) ^ sw], a3 = aq[(4 * r + 3) ^ sw];
    const uint32_t q[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
    const int al[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
    const int ah[8] = {a2.x, a2.y, a2.z, a2.w, a3.x, a3.y, a3.z, a3.w};
    int lo0 = 0, lo1 = 0, hi0 = 0, hi1 = 0;   // two chains each: shorter dependency paths
#pragma unroll
    for (int i = 0; i < 8; i += 2) {
      lo0 = __dp4a((int)(q[i] & 0x0f0f0f0fu), al[i], lo0);
      lo1 = __dp4a((int)(q[i + 1] & 0x0f0f0f0fu), al[i + 1], lo1);
      hi0 = dp4a_us(q[i] & 0xf0f0f0f0u, ah[i], hi0);
      hi1 = dp4a_us(q[i + 1] & 0xf0f0f0f0u, ah[i + 1], hi1);
    }
    const uint32_t scw = r < 2 ? sc_lo : sc_hi, mnw = r < 2 ? mn_lo : mn_hi;
    const int sh = 16 * (r & 1);
    const int bs_lo = (int)(short)(bw[2 * r] & 0xffff) + (bw[2 * r] >> 16);
    const int bs_hi = (int)(short)(bw[2 * r + 1] & 0xffff) + (bw[2 * r + 1] >> 16);
    isum += (int)((scw >> sh) & 0xff) * (lo0 + lo1) + (int)((scw >> (sh + 8)) & 0xff) * ((hi0 + hi1) >> 4);
    msum += (int)((mnw >> sh) & 0xff) * bs_lo + (int)((mnw >> (sh + 8)) & 0xff) * bs_hi;
  }
  const float dx = x.d[e0 / QK_K];
  const float d = h2f((uint16_t)(h.x & 0xffffu)), dmin = h2f((uint16_t)(h.x >> 16));
  return __fmaf_rn(__fmul_rn(dx, d), (float)isum, -__fmul_rn(__fmul_rn(dx, dmin), (float)msum));
}

// the register-resident block-value functions above, fed from the shared copy
template <int T>
__device__ __forceinline__ void fill_act_from_smem(Act256& x, const ActSmem& s, int e0) {
  const int4* q = reinterpret_cast<const int4*>(s.qs + e0);
  const int sw = act_swizzle(e0);
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const int4 v = q[i ^ sw];
    x.a[4 * i + 0] = v.x; x.a[4 * i + 1] = v.y; x.a[4 * i + 2] = v.z; x.a[4 * i + 3] = v.w;
  }
  if constexpr (is_k_type(T)) {
    const int4* b = reinterpret_cast<const int4*>(s.bs + e0 / 16);
    const int4 b0 = b[0], b1 = b[1];
    const int w[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int lo = (int)(short)(w[j] & 0xffff), hi = w[j] >> 16;
      x.bs[j] = lo + hi;
      x.bs16[2 * j] = lo;
      x.bs16[2 * j + 1] = hi;
    }
    x.d[0] = s.d[e0 / QK_K];
  } else {
    const float4* dd = reinterpret_cast<const float4*>(s.d + e0 / 32);
    const float4 d0 = dd[0], d1 = dd[1];
    x.d[0] = d0.x; x.d[1] = d0.y; x.d[2] = d0.z; x.d[3] = d0.w;
    x.d[4] = d1.x; x.d[5] = d1.y; x.d[6] = d1.z; x.d[7] = d1.w;
  }
}

__host__ __device__ constexpr int act_smem_bytes(bool kq, int K) {
  // qs | bsums (K-quants) | d ; each part 16-byte rounded
  return ((K + 15) / 16) * 16 + (kq ? ((K / 8 + 15) / 16) * 16 : 0) + (((kq ? K / 256 : K / 32) * 4 + 15) / 16) * 16;
}

template <int T, int STAGES>
__host__ __device__ constexpr int warp_bytes3() {
  return STAGES * ROWS_PER_STAGE * Geo2<T>::CB + ((STAGES * 8 + STAGES * 8 + 15) / 16) * 16;  // ring + barriers + (task, chunk)
}

// NCOLS > 1: the same rows against NCOLS activation columns (plain outputs only): the weights of a stage
// are decoded once per column from shared memory, every column keeps its own f32 chain
// JOIN: the launch waits for / raises a join by peer stores (row-sharded sessions); compiled apart so that the
// one-GPU kernels carry none of it
template <int T, int STAGES, int WARPS, int MINB, bool ARGMAX, int NCOLS = 1, bool JOIN = false>
__global__ void __launch_bounds__(WARPS * 32, MINB)
gemv3_kernel(const GemvArgs p) {
  static_assert(NCOLS == 1 || !ARGMAX, "the fused argmax is a one-column path");
  constexpr int CB = Geo2<T>::CB;
  constexpr bool KQ = is_k_type(T);
  constexpr int SPAN = CB / 8;
  extern __shared__ __align__(128) uint8_t smem3[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int act_bytes = act_smem_bytes(KQ, p.K);
  uint8_t* ring = smem3 + NCOLS * act_bytes + (size_t)warp * warp_bytes3<T, STAGES>();
  uint64_t* bars = reinterpret_cast<uint64_t*>(ring + STAGES * ROWS_PER_STAGE * CB);
  int* meta = reinterpret_cast<int*>(bars + STAGES);  // 2 ints per stage: task, chunk

  const int nchunks = p.K / CHUNK;
  const int nt0 = (p.M + ROWS_PER_STAGE - 1) / ROWS_PER_STAGE;
  const int nt1 = (p.M2 + ROWS_PER_STAGE - 1) / ROWS_PER_STAGE;
  const int nt2 = (p.M3 + ROWS_PER_STAGE - 1) / ROWS_PER_STAGE;
  const int ntasks = nt0 + nt1 + nt2;

  pdl_trigger();
  // the join descriptors are constants of the session: fetched now, while the first weight copies start
  JoinIn ji{};
  char* jo_base = nullptr;
  int64_t jo_offset = 0;
  if constexpr (JOIN) {
    if (p.join_in) ji = *p.join_in;
    if (p.join_out) {
      jo_offset = p.join_out->out_offset;
      if (lane < p.join_out->world) jo_base = p.join_out->base[lane];
    }
  }
  if (lane == 0) {
#pragma unroll
    for (int s = 0; s < STAGES; ++s) mbar_init(bars + s, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  __syncwarp();

  const int total_warps = gridDim.x * WARPS;
  int iss_task = blockIdx.x * WARPS + warp, iss_chunk = 0;
  bool drained = iss_task >= ntasks;
  auto issue_next = [&](int slot) {
    if (!drained && iss_chunk == nchunks) {
      int t = 0;
      if (lane == 0) t = atomicAdd(p.sched, 1);
      iss_task = __shfl_sync(0xffffffffu, t, 0) + total_warps;
      iss_chunk = 0;
      drained = iss_task >= ntasks;
    }
    if (lane == 0) {
      meta[2 * slot] = drained ? -1 : iss_task;
      meta[2 * slot + 1] = iss_chunk;
      if (!drained) {
        const int seg = iss_task < nt0 ? 0 : (iss_task < nt0 + nt1 ? 1 : 2);
        const int lt = iss_task - (seg == 0 ? 0 : (seg == 1 ? nt0 : nt0 + nt1));
        const uint8_t* wbase = seg == 0 ? p.W : (seg == 1 ? p.W2 : p.W3);
        const int mseg = seg == 0 ? p.M : (seg == 1 ? p.M2 : p.M3);
        uint8_t* dst = ring + (size_t)slot * ROWS_PER_STAGE * CB;
        mbar_expect_tx(bars + slot, ROWS_PER_STAGE * CB);
#pragma unroll
        for (int r = 0; r < ROWS_PER_STAGE; ++r) {
          const int row = min(lt * ROWS_PER_STAGE + r, mseg - 1);
          bulk_g2s(dst + r * CB, wbase + (size_t)row * p.row_bytes + (size_t)iss_chunk * CB, CB, bars + slot);
        }
      }
    }
    if (!drained) ++iss_chunk;
  };

  // the weight copies do not depend on the previous kernel: start them first
#pragma unroll
  for (int s = 0; s < STAGES; ++s) issue_next(s);
  pdl_wait();
  // a joined input vector: every peer's rows must have landed before the first read
  bool joined_in = false;
  if constexpr (JOIN) {
    if (p.join_in) {
      joined_in = true;
      join_wait(ji, p.status);
    }
  }

  // this column's quantized activations in shared memory for the whole CTA: copied from the planes, or
  // (fused prologue) normalised and quantized here from the f32 vector
  ActSmem x;   // column 0; column j lies j * act_bytes further
#pragma unroll 1
  for (int col = 0; col < NCOLS; ++col) {
    uint8_t* abase = smem3 + (size_t)col * act_bytes;
    int8_t* sq = reinterpret_cast<int8_t*>(abase);
    int16_t* sb = reinterpret_cast<int16_t*>(abase + ((p.K + 15) / 16) * 16);
    float* sd = reinterpret_cast<float*>(abase + ((p.K + 15) / 16) * 16 + (KQ ? ((p.K / 8 + 15) / 16) * 16 : 0));
    bool fused = false;
    if constexpr (KQ && NCOLS == 1) {
      if (p.pro_x) {
        fused = true;
        // rows written by peers are read past the L1 (ld.cg): a line of an earlier read may still sit there
        auto ldx = [&](const float* a) { return JOIN && joined_in ? __ldcg(a) : __ldg(a); };
        auto ldx4 = [&](const float* a) { return JOIN && joined_in ? __ldcg(reinterpret_cast<const float4*>(a)) : __ldg(reinterpret_cast<const float4*>(a)); };
        float scale = 1.0f;
        if (p.pro_w) {
          // rms_norm (src/emel/text/generator/detail.hpp:2735-2756): f64 sum of the f32 squares
          __shared__ double s_part[WARPS];
          double ss = 0.0;
          for (int i = threadIdx.x; i < p.K; i += WARPS * 32) {
            const float v = ldx(p.pro_x + i);
            ss += (double)__fmul_rn(v, v);
          }
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
          if (lane == 0) s_part[warp] = ss;
          __syncthreads();
          double total = 0.0;
#pragma unroll
          for (int w = 0; w < WARPS; ++w) total += s_part[w];
          const float mean = (float)(total / (double)p.K);
          scale = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(mean, p.pro_eps)));
        }
        for (int blk = warp; blk < p.K / QK_K; blk += WARPS) {
          float v[8];
          const int e0 = blk * QK_K + 8 * lane;
          const float4 x0 = ldx4(p.pro_x + e0), x1 = ldx4(p.pro_x + e0 + 4);
          const float xs[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
          if (p.pro_w) {
            const float4 w0 = __ldg(reinterpret_cast<const float4*>(p.pro_w + e0)), w1 = __ldg(reinterpret_cast<const float4*>(p.pro_w + e0) + 1);
            const float ws[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = __fmul_rn(__fmul_rn(xs[i], scale), ws[i]);
          } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = xs[i];
          }
          uint32_t lo, hi; int bs16; float dq;
          q8_k_block_warp(v, lane, lo, hi, bs16, dq);
          const int unit = blk * 16 + ((lane >> 1) ^ (blk & 7));        // the swizzled 16-byte unit of elements 8*lane..
          *reinterpret_cast<uint2*>(sq + unit * 16 + (lane & 1) * 8) = make_uint2(lo, hi);
          if ((lane & 1) == 0) sb[blk * 16 + (lane >> 1)] = (int16_t)bs16;
          if (lane == 0) sd[blk] = dq;
        }
      }
    }
    if (!fused) {
      const int64_t gcol = p.col0 + col;
      const int4* gq = reinterpret_cast<const int4*>(p.act.qs + gcol * p.act.col_stride_qs);
      // planes written by peers are read past the L1 (ld.cg): a line of an earlier read may still sit there
      for (int i = threadIdx.x; i < p.K / 16; i += WARPS * 32)
        reinterpret_cast<int4*>(sq)[i ^ ((i >> 4) & 7)] = JOIN && joined_in ? __ldcg(gq + i) : __ldg(gq + i);
      if constexpr (KQ) {
        const int4* gb = reinterpret_cast<const int4*>(p.act.bsums + gcol * p.act.col_stride_bs);
        for (int i = threadIdx.x; i < p.K / 128; i += WARPS * 32) reinterpret_cast<int4*>(sb)[i] = JOIN && joined_in ? __ldcg(gb + i) : __ldg(gb + i);
      }
      const float* gd = p.act.d + gcol * p.act.col_stride_d;
      const int nd = KQ ? p.K / QK_K : p.K / 32;
      for (int i = threadIdx.x; i < nd; i += WARPS * 32) sd[i] = JOIN && joined_in ? __ldcg(gd + i) : __ldg(gd + i);
    }
    if (col == 0) {
      x.qs = sq;
      x.bs = sb;
      x.d = sd;
    }
  }
  __syncthreads();

  const int r4 = lane >> 3, b = lane & 7;
  float accs[NCOLS];
#pragma unroll
  for (int j = 0; j < NCOLS; ++j) accs[j] = 0.0f;
  float best = -INFINITY;
  int best_i = 0x7fffffff;
  uint32_t phase = 0;
  int slot_c = 0;
  bool failed = false;

  for (;;) {
    const int task = meta[2 * slot_c], c = meta[2 * slot_c + 1];
    if (task < 0) break;
    {
      int spins = 0;
      bool ok = false;
      unsigned long long t_start = 0;
      while (!(ok = mbar_try_wait(bars + slot_c, (phase >> slot_c) & 1u)) && ++spins < kWaitLimit) {
        if ((spins & 255) == 0) {
          unsigned long long now;
          asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
          if (t_start == 0) t_start = now;
          else if (now - t_start > kWaitLimitNs) break;
        }
      }
      if (!__all_sync(0xffffffffu, ok)) { failed = true; break; }
      phase ^= 1u << slot_c;
    }
    if (c == 0) {
#pragma unroll
      for (int j = 0; j < NCOLS; ++j) accs[j] = 0.0f;
    }
    const uint8_t* st = ring + (size_t)slot_c * ROWS_PER_STAGE * CB + r4 * CB + b * SPAN;
    const int e0 = c * CHUNK + 256 * b;
#pragma unroll
    for (int j = 0; j < NCOLS; ++j) {
      ActSmem xj;
      xj.qs = x.qs + (size_t)j * act_bytes;
      xj.bs = reinterpret_cast<const int16_t*>(reinterpret_cast<const uint8_t*>(x.bs) + (size_t)j * act_bytes);
      xj.d = reinterpret_cast<const float*>(reinterpret_cast<const uint8_t*>(x.d) + (size_t)j * act_bytes);
      float acc = accs[j];
    if constexpr (T == T_Q4_K) {
      const float bv = q4_k_block_value_s(st, xj, e0);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc = __fadd_rn(acc, __shfl_sync(0xffffffffu, bv, (lane & ~7) + i));
    } else {
      Act256 xr;
      fill_act_from_smem<T>(xr, xj, e0);
      if constexpr (T == T_Q6_K) {
        const float bv = q6_k_block_value(st, xr);
#pragma unroll
        for (int i = 0; i < 8; ++i) acc = __fadd_rn(acc, __shfl_sync(0xffffffffu, bv, (lane & ~7) + i));
      } else {
        float bv[8];
        if constexpr (T == T_Q8_0) q8_0_block_values(st, xr, bv);
        else q4_0_block_values(st, xr, bv);
#pragma unroll
        for (int g = 0; g < 8; ++g)
#pragma unroll
          for (int i = 0; i < 8; ++i) acc = __fadd_rn(acc, __shfl_sync(0xffffffffu, bv[i], (lane & ~7) + g));
      }
    }
      accs[j] = acc;
    }
    const float acc = accs[0];
    if (c == nchunks - 1) {
      const int seg = task < nt0 ? 0 : (task < nt0 + nt1 ? 1 : 2);
      const int lt = task - (seg == 0 ? 0 : (seg == 1 ? nt0 : nt0 + nt1));
      const int mseg = seg == 0 ? p.M : (seg == 1 ? p.M2 : p.M3);
      float* yseg = seg == 0 ? p.y : (seg == 1 ? p.y2 : p.y3);
      const int row = lt * ROWS_PER_STAGE + r4;
      bool plain = true;
      if constexpr (!ARGMAX && NCOLS == 1) {
        if (p.rope_cos) {
          // rows 2p, 2p+1 of a head are one rotation pair and sit in neighbouring 8-lane groups of this warp
          // (apply_rope_pairing, src/emel/text/generator/detail.hpp:2905-2936; KV rows rounded to f16, :3294-3332)
          plain = false;
          const float other = __shfl_sync(0xffffffffu, acc, ((r4 ^ 1) << 3));
          if (b == 0 && row < mseg) {
            const int hd = p.rope_head_dim, head = row / hd, d = row - head * hd;
            const int rseg = seg + p.rope_seg0;    // 0: query rows, 1: key rows, 2: value rows
            float out = acc;
            if (rseg < 2 && d < p.rope_rot_dim) {
              const int pos = *p.rope_pos, pairs = p.rope_rot_dim >> 1;
              const float cs = p.rope_cos[(int64_t)pos * pairs + (d >> 1)], sn = p.rope_sin[(int64_t)pos * pairs + (d >> 1)];
              out = (d & 1) ? __fadd_rn(__fmul_rn(other, sn), __fmul_rn(acc, cs)) : __fsub_rn(__fmul_rn(acc, cs), __fmul_rn(other, sn));
            }
            if (rseg == 0) yseg[row] = out;
            else {
              __half* cache = rseg == 1 ? p.rope_kcache : p.rope_vcache;
              cache[(int64_t)head * p.rope_cache_head_stride + (int64_t)(*p.rope_pos) * hd + d] = __float2half_rn(out);
            }
          }
        }
      }
      if constexpr (JOIN) {
        if (p.join_out) {
          // this rank's rows go to every rank's copy of the vector: the four rows of the task are collected and
          // lanes 0 .. world-1 store them to one rank each (row counts are multiples of four in a sharded session)
          plain = false;
          float o = acc;
          if (b == 0 && row < mseg && p.residual) o = __fadd_rn(p.residual[row], acc);
          const float4 o4 = make_float4(__shfl_sync(0xffffffffu, o, 0), __shfl_sync(0xffffffffu, o, 8),
                                        __shfl_sync(0xffffffffu, o, 16), __shfl_sync(0xffffffffu, o, 24));
          const int row0 = lt * ROWS_PER_STAGE;
          if (jo_base && row0 + ROWS_PER_STAGE <= mseg)
            *reinterpret_cast<float4*>(jo_base + jo_offset + (int64_t)row0 * 4) = o4;
        }
      }
      if (plain && row < mseg) {
        if constexpr (ARGMAX) {
          if (acc > best || best_i == 0x7fffffff) { best = acc; best_i = row; }
        } else if (b == 0) {
#pragma unroll
          for (int j = 0; j < NCOLS; ++j) {
            const size_t o = (size_t)row * p.ldy + p.col0 + j;
            yseg[o] = (p.residual && seg == 0) ? __fadd_rn(p.residual[o], accs[j]) : accs[j];
          }
        }
      }
    }
    __syncwarp();            // the stage is free
    issue_next(slot_c);      // refill it right away
    __syncwarp();
    slot_c = slot_c + 1 == STAGES ? 0 : slot_c + 1;
  }
  if (failed && lane == 0 && p.status) atomicExch(p.status, 1);

  constexpr bool kJoins = JOIN;
  if (kJoins && p.join_out) __threadfence_system();   // this thread's stores to the peers, before the block is counted
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(p.sched + 1, 1) == (int)gridDim.x - 1) {
      p.sched[0] = 0;
      p.sched[1] = 0;
      __threadfence();
      if (kJoins && p.join_out) join_raise(*p.join_out);
    }
  }

  if constexpr (ARGMAX) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
      if (oi != 0x7fffffff && (best_i == 0x7fffffff || ov > best || (ov == best && oi < best_i))) { best = ov; best_i = oi; }
    }
    __shared__ float sv[WARPS];
    __shared__ int si[WARPS];
    if (lane == 0) { sv[warp] = best; si[warp] = best_i; }
    __syncthreads();
    if (threadIdx.x == 0) {
      float bvv = sv[0]; int bi = si[0];
      for (int w = 1; w < WARPS; ++w)
        if (si[w] != 0x7fffffff && (bi == 0x7fffffff || sv[w] > bvv || (sv[w] == bvv && si[w] < bi))) { bvv = sv[w]; bi = si[w]; }
      p.part_val[blockIdx.x] = bvv;
      p.part_idx[blockIdx.x] = bi;
    }
  }
}

// ---------------------------------------------------------------- launch
constexpr int kWarps2 = 4;

template <int T> constexpr int stages_for() { return (T == T_Q4_K || T == T_Q4_0) ? 4 : 3; }

template <int T, int NCOLS, int RP, bool ARGMAX>
cudaError_t launch2(const GemvArgs& a, int sm_count, cudaStream_t st, int* grid_out) {
  constexpr int STAGES = stages_for<T>();
  constexpr size_t smem = (size_t)kWarps2 * warp_bytes2<T, STAGES>();
  auto kern = gemv2_kernel<T, NCOLS, RP, STAGES, kWarps2, ARGMAX>;
  // per instantiation and host thread (one context, one lane per thread), one bit per device
  static thread_local unsigned configured = 0;
  int dev = 0;
  cudaGetDevice(&dev);
  if (!(configured & (1u << (dev & 31)))) {
    const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    configured |= 1u << (dev & 31);
  }
  const int rows_per_task = ROWS_PER_STAGE * RP;
  const int ntasks = (a.M + rows_per_task - 1) / rows_per_task + (a.M2 + rows_per_task - 1) / rows_per_task +
                     (a.M3 + rows_per_task - 1) / rows_per_task;
  int per_sm = (int)((220 * 1024) / smem);
  if (per_sm < 1) per_sm = 1;
  if (per_sm > 6) per_sm = 6;
  int grid = (ntasks + kWarps2 - 1) / kWarps2;
  if (grid > sm_count * per_sm) grid = sm_count * per_sm;
  if (ARGMAX && grid > kMaxArgmaxParts) grid = kMaxArgmaxParts;
  if (grid_out) *grid_out = grid;
  return launch_kernel(kern, dim3(grid), dim3(kWarps2 * 32), smem, st, a.pdl != 0, a);
}

// third generation: one column (or the argmax head), activations in shared memory
template <int T, int STAGES, int WARPS, int MINB, bool ARGMAX, int NCOLS = 1, bool JOIN = false>
cudaError_t launch3(const GemvArgs& a, int sm_count, cudaStream_t st, int* grid_out) {
  auto kern = gemv3_kernel<T, STAGES, WARPS, MINB, ARGMAX, NCOLS, JOIN>;
  const size_t smem = (size_t)NCOLS * act_smem_bytes(is_k_type(T), a.K) + (size_t)WARPS * warp_bytes3<T, STAGES>();
  // Per instantiation, host thread (one context, one lane per thread) and device: the attribute is set once,
  // and the CTAs per SM are remembered for the last few shared-memory sizes (matrices of different K alternate
  // on one instantiation inside a decode step).
  struct Cache {
    bool attr = false;
    size_t smem[4] = {};
    int per_sm[4] = {};
    int next = 0;
  };
  static thread_local Cache caches[32];
  int dev = 0;
  cudaGetDevice(&dev);
  Cache& c = caches[dev & 31];
  if (!c.attr) {
    const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    if (e != cudaSuccess) return e;
    c.attr = true;
  }
  int per_sm = 0;
  for (int i = 0; i < 4; ++i)
    if (c.smem[i] == smem && c.per_sm[i] > 0) per_sm = c.per_sm[i];
  if (per_sm == 0) {
    const cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, WARPS * 32, smem);
    if (e != cudaSuccess) return e;
    if (per_sm < 1) return cudaErrorInvalidConfiguration;
    c.smem[c.next] = smem;
    c.per_sm[c.next] = per_sm;
    c.next = (c.next + 1) & 3;
  }
  const int ntasks = (a.M + ROWS_PER_STAGE - 1) / ROWS_PER_STAGE + (a.M2 + ROWS_PER_STAGE - 1) / ROWS_PER_STAGE +
                     (a.M3 + ROWS_PER_STAGE - 1) / ROWS_PER_STAGE;
  int grid = (ntasks + WARPS - 1) / WARPS;
  if (grid > sm_count * per_sm) grid = sm_count * per_sm;
  if (ARGMAX && grid > kMaxArgmaxParts) grid = kMaxArgmaxParts;
  if (grid_out) *grid_out = grid;
  return launch_kernel(kern, dim3(grid), dim3(WARPS * 32), smem, st, a.pdl != 0, a);
}

template <int T, bool ARGMAX, bool JOIN = false>
cudaError_t launch3_cfg(const GemvArgs& a, int sm_count, cudaStream_t st, int* grid_out) {
  constexpr bool kLight = T == T_Q4_K || T == T_Q4_0;  // 64 registers: 32 warps per SM; the others 16
  constexpr int kWarpsPerSm = kLight ? 32 : 16;
  // few rows: smaller CTAs, so that every SM gets about the same number of 4-row tasks
  const int ntasks = (a.M + ROWS_PER_STAGE - 1) / ROWS_PER_STAGE + (a.M2 + ROWS_PER_STAGE - 1) / ROWS_PER_STAGE +
                     (a.M3 + ROWS_PER_STAGE - 1) / ROWS_PER_STAGE;
  // With the normalisation in the prologue every CTA normalises and quantizes the whole vector before its first
  // product: eight warps share that work, whatever the task count (with two-warp CTAs the grouped Q/K/V launch of
  // the 8B shape spent half its time there: the decode step went from 441 to 468 tok/s with this rule)
  const bool norm_prologue = a.pro_x && a.pro_w;
  if constexpr (kLight && !ARGMAX) {
    // many tasks and a long vector: one CTA of 32 warps per SM normalises once where four CTAs of eight warps did it
    // four times (70B shape, K = 8192: 84.8 -> 86.0 tok/s; at K = 4096 the eight-warp CTAs are faster, 469 against 458)
    if (norm_prologue && ntasks >= 32 * sm_count && a.K >= 8192) return launch3<T, 1, 32, 1, ARGMAX, 1, JOIN>(a, sm_count, st, grid_out);
    if (norm_prologue && ntasks >= 32 * sm_count) return launch3<T, 1, 16, 2, ARGMAX, 1, JOIN>(a, sm_count, st, grid_out);
  }
  if (ntasks >= 8 * 3 * sm_count || ARGMAX || (norm_prologue && ntasks >= 4 * 3 * sm_count))
    return launch3<T, 1, 8, kWarpsPerSm / 8, ARGMAX, 1, JOIN>(a, sm_count, st, grid_out);
  if (ntasks >= 4 * 3 * sm_count) return launch3<T, 1, 4, kWarpsPerSm / 4, ARGMAX, 1, JOIN>(a, sm_count, st, grid_out);
  // about one task per warp: keep the whole row group of a warp in flight (2 chunks), or a deeper ring for long rows;
  // eight warps per CTA here too, so that eight tasks share one copy of the activations (8B shape: 473 -> 478 tok/s;
  // the same change for the middle range of task counts cost the 70B shape 4 %, so that range keeps four warps)
  if constexpr (kLight) {
    if (a.K / CHUNK >= 4 && !norm_prologue) return launch3<T, 4, 8, 1, ARGMAX, 1, JOIN>(a, sm_count, st, grid_out);
    return launch3<T, 2, 8, 2, ARGMAX, 1, JOIN>(a, sm_count, st, grid_out);
  } else {
    // the wider block formats (1680 / 2176 bytes per row and stage) keep two-warp CTAs: eight four-stage rings do
    // not fit in shared memory
    if (norm_prologue) return launch3<T, 2, 8, 1, ARGMAX, 1, JOIN>(a, sm_count, st, grid_out);
    if (a.K / CHUNK >= 4) return launch3<T, 4, 2, 3, ARGMAX, 1, JOIN>(a, sm_count, st, grid_out);
    return launch3<T, 2, 2, 4, ARGMAX, 1, JOIN>(a, sm_count, st, grid_out);
  }
}

template <int T>
cudaError_t launch_type2(GemvArgs a, int ncols, bool argmax, int sm_count, cudaStream_t st, int* launches, int* grid_out) {
  if (argmax) {
    ++*launches;
    return launch3_cfg<T, true>(a, sm_count, st, grid_out);
  }
  cudaError_t e = cudaSuccess;
  int done = 0;
  while (done < ncols && e == cudaSuccess) {
    GemvArgs b = a;
    b.col0 = a.col0 + done;
    const int left = ncols - done;
    // several columns: the third-generation kernel while their activations fit beside the rings
    const bool multi3 = !b.pro_x && !b.rope_cos;
    const size_t act1 = (size_t)act_smem_bytes(is_k_type(T), a.K);
    if (left >= 8 && multi3 && 8 * act1 <= 64 * 1024) { e = launch3<T, 1, 8, 2, false, 8>(b, sm_count, st, grid_out); done += 8; }
    else if (left >= 4 && multi3 && 4 * act1 <= 64 * 1024) { e = launch3<T, 1, 8, 2, false, 4>(b, sm_count, st, grid_out); done += 4; }
    else if (left >= 2 && multi3 && 2 * act1 <= 64 * 1024) { e = launch3<T, 1, 8, 2, false, 2>(b, sm_count, st, grid_out); done += 2; }
    else if (left >= 8) { e = launch2<T, 8, 1, false>(b, sm_count, st, grid_out); done += 8; }
    else if (left >= 4) { e = launch2<T, 4, 1, false>(b, sm_count, st, grid_out); done += 4; }
    else if (left >= 2) { e = launch2<T, 2, 1, false>(b, sm_count, st, grid_out); done += 2; }
    else {
      const bool join = b.join_in != nullptr || b.join_out != nullptr;
      if constexpr (is_k_type(T)) e = join ? launch3_cfg<T, false, true>(b, sm_count, st, grid_out) : launch3_cfg<T, false>(b, sm_count, st, grid_out);
      else e = join ? cudaErrorInvalidValue : launch3_cfg<T, false>(b, sm_count, st, grid_out);
      done += 1;
    }
    ++*launches;
  }
  return e;
}

}  // namespace

bool gemv_prologue_supported(int type, const void* w, int64_t row_bytes, int K) {
  return is_k_type(type) && (K % CHUNK) == 0 && (reinterpret_cast<uintptr_t>(w) % 16) == 0 &&
         (row_bytes % 16) == 0;
}

// the streaming path for K % 2048 == 0 and 16-byte aligned rows; the caller runs the
// argmax finishing kernel over *grid_out candidates
cudaError_t launch_gemv_stream2(int type, const GemvArgs& a, int ncols, bool argmax, int sm_count, cudaStream_t st,
                                int* launches, int* grid_out) {
  switch (type) {
    case T_Q4_K: return launch_type2<T_Q4_K>(a, ncols, argmax, sm_count, st, launches, grid_out);
    case T_Q6_K: return launch_type2<T_Q6_K>(a, ncols, argmax, sm_count, st, launches, grid_out);
    case T_Q8_0: return launch_type2<T_Q8_0>(a, ncols, argmax, sm_count, st, launches, grid_out);
    case T_Q4_0: return launch_type2<T_Q4_0>(a, ncols, argmax, sm_count, st, launches, grid_out);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace emelb
