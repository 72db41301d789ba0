// Q4_K x Q8_K matrix product for many columns (prompt processing) on the
// Blackwell tensor cores: tcgen05.mma kind::i8 with int32 accumulators in TMEM.
//
// What is computed is exactly the reference's per-super-block value,
//   fma(d*dx, isum, -(dmin*dx)*msum),   isum = sum_j sc_j * dot_j(q, x),
//   msum = sum_j m_j * bsum_j           (src/emel/kernel/x86_64/actions.hpp:859-866)
// added in ascending block order, so the result equals the mat-vec kernels' (and
// the x86 AVX2 route's) bit for bit.  The integer part runs on the tensor cores:
//   * a 6-bit scale times a 4-bit quant does not fit int8, so sc_j = 8*hi_j + lo_j
//     and two int8 operands are built per row, q*lo_j and q*hi_j (each <= 105);
//     isum = D_lo + 8*D_hi, exact in int32;
//   * one MMA has K = 32 = one sub-block, 16 MMAs (8 sub-blocks x {lo, hi}) cover
//     a super-block of 256; then the accumulators are read back (tcgen05.ld) and
//     folded into f32 registers with the block's scales — the float chain stays on
//     the CUDA cores because its order and roundings are part of the contract.
//
// CTA = 128 rows x 128 columns, 21 warps:
//   warps 0-3   producers: the 128 GGUF blocks of a super-block column arrive by
//               cp.async.bulk (one 144-byte copy per row) in a raw staging buffer;
//               thread p expands row p into the two int8 operands, and the warp
//               copies 32 columns' activations with cp.async (8 columns x 64
//               contiguous bytes per instruction), both into the canonical
//               no-swizzle K-major layout (8 rows x 16 bytes core matrices)
//   warp  4     allocates TMEM, issues the MMAs, commits to an mbarrier
//   warps 5-20  epilogue: four warps per TMEM lane quarter, 32 columns each
// Two shared-memory stages and two TMEM accumulator pairs (2 x 256 columns) let
// producers, tensor cores and epilogue work on different super-blocks at once.
// Every mbarrier wait is bounded; on a timeout the CTA raises the status word,
// stops issuing, and still frees its TMEM.
#include <cuda_runtime.h>
#include <stdint.h>

#include "common.cuh"
#include "kernels.h"

namespace emelb {
namespace {

constexpr int BM = 128, BN = 128;
constexpr int kProducerThreads = 128;
constexpr int kMmaWarp = 4;
constexpr int kEpilogueWarp0 = 5;
constexpr int kThreads = 21 * 32;
constexpr int kEpilogueWarps = 16;
constexpr int kStages = 2;

// shared memory map (bytes)
constexpr int kOperandBytes = BM * 256;                 // one int8 operand tile of a super-block: 32 KB
constexpr int kChunkStride = (BM / 8) * 128;            // next 16-byte K chunk: 2048 B (leading byte offset)
constexpr int kGroupStride = 128;                       // next 8-row core matrix (stride byte offset)
constexpr int kStageBytes = 3 * kOperandBytes           // A_lo, A_hi, B
                            + BM * 16                   // row meta {d, dmin, mins[8]}
                            + BN * 16                   // column meta: 8 pair sums (int16)
                            + BN * 4;                   // column scale dx
constexpr int kOffAlo = 0, kOffAhi = kOperandBytes, kOffB = 2 * kOperandBytes, kOffRowMeta = 3 * kOperandBytes,
              kOffColMeta = kOffRowMeta + BM * 16, kOffDx = kOffColMeta + BN * 16;
constexpr int kRawBytes = BM * Q4_K_BYTES;              // raw GGUF blocks of one super-block column: 18,432 B
constexpr int kBarBytes = 64;                           // full[2], tmem_full[2], epi_done[2], raw_full, tmem base, abort
constexpr int kSmemBytes = kStages * kStageBytes + kRawBytes + kBarBytes + 128;  // + alignment slack

constexpr int kWaitSpins = 1 << 22;
constexpr unsigned long long kWaitNs = 2000000000ull;  // 2 s

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
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

// bounded wait; false when it gave up or another role already raised the abort flag
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  unsigned long long t0 = 0;
  for (int spins = 0; spins < kWaitSpins; ++spins) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((spins & 63) == 63) {
      if (*abort_flag) return false;
      unsigned long long now;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
      if (t0 == 0) t0 = now;
      else if (now - t0 > kWaitNs) break;
    }
  }
  *abort_flag = 1;
  return false;
}

__device__ __forceinline__ uint64_t operand_desc(uint32_t saddr) {
  // K-major, no swizzle: 14-bit fields in 16-byte units; descriptor version 1 (sm_100)
  uint64_t d = 0;
  d |= (uint64_t)((saddr >> 4) & 0x3fffu);
  d |= (uint64_t)((kChunkStride >> 4) & 0x3fffu) << 16;   // leading byte offset: between the two 16-byte K chunks
  d |= (uint64_t)((kGroupStride >> 4) & 0x3fffu) << 32;   // stride byte offset: between 8-row groups
  d |= (uint64_t)1 << 46;
  return d;
}

// instruction descriptor: D = s32, A = B = signed 8-bit, both K-major, N = 128, M = 128
constexpr uint32_t kInstrDesc = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);

__device__ __forceinline__ void mma_i8(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(da), "l"(db), "r"(kInstrDesc), "r"(accumulate)
      : "memory");
}

__device__ __forceinline__ void mma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void tmem_ld8(uint32_t taddr, uint32_t (&v)[8]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7])
               : "r"(taddr)
               : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(dst)),
               "l"(src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

struct GemmArgs {
  const uint8_t* W;
  int64_t row_bytes;
  int M, K, N;
  ActPlanes act;
  int col0;
  float* y;
  int64_t ldy;
  int* status;
};

__global__ void __launch_bounds__(kThreads, 1) gemm_q4k_tc_kernel(const GemmArgs p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
  uint8_t* raw = smem + kStages * kStageBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(raw + kRawBytes);
  uint64_t* full = bars;            // [2] producers -> MMA: operands of a super-block are in shared memory
  uint64_t* tmem_full = bars + 2;   // [2] MMA -> epilogue: the accumulator pair holds a finished super-block
  uint64_t* epi_done = bars + 4;    // [2] epilogue -> producers: stage and accumulator pair are free again
  uint64_t* raw_full = bars + 6;    // bulk copies -> producers: the raw blocks of the next super-block landed
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 7);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(full + s, kProducerThreads);
      mbar_init(tmem_full + s, 1);
      mbar_init(epi_done + s, kEpilogueWarps);
    }
    mbar_init(raw_full, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == kMmaWarp) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;

  const int mt = (p.M + BM - 1) / BM, nt = (p.N + BN - 1) / BN, ntiles = mt * nt, nkb = p.K / QK_K;

  if (warp < 4) {
    // ---------------------------------------------------------------- producers
    const int t = threadIdx.x;  // row t of the weight tile; column t for the per-column scales
    const uint32_t core_off = (uint32_t)(t >> 3) * kGroupStride + (uint32_t)(t & 7) * 16;
    // raw copy of row t's block of iteration (tile, kb); thread 0 also arms the barrier
    auto issue_raw = [&](int tile, int kb) {
      const int tm = tile / nt;
      const int row = min(tm * BM + t, p.M - 1);          // out-of-range rows/columns repeat the last one; never stored
      if (t == 0) mbar_arrive_expect_tx(raw_full, kRawBytes);
      bulk_g2s(raw + t * Q4_K_BYTES, p.W + (size_t)row * p.row_bytes + (size_t)kb * Q4_K_BYTES, Q4_K_BYTES, raw_full);
    };
    // One flat loop over (tile, super-block).  The 128 producers meet at a named barrier every
    // iteration, so nobody leaves early: a wait that gave up only skips work, and the loop ends
    // for everyone at the abort check right after the barrier.
    int it = 0, tile = blockIdx.x, kb = 0;
    if (tile < ntiles) issue_raw(tile, 0);
    for (; tile < ntiles; ++it) {
      const int tn = tile % nt;
      const int s = it & 1;
      // this row's 144 raw bytes -> registers, then the staging buffer is free for the next copy
      bool ok = mbar_wait(raw_full, it & 1, abort_flag);
      uint4 blk[9];
#pragma unroll
      for (int i = 0; i < 9; ++i) blk[i] = *reinterpret_cast<const uint4*>(raw + t * Q4_K_BYTES + 16 * i);
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (*abort_flag) break;
      int ntile = tile, nkbi = kb + 1;
      if (nkbi == nkb) { nkbi = 0; ntile += gridDim.x; }
      if (ntile < ntiles) issue_raw(ntile, nkbi);
      ok = ok && mbar_wait(epi_done + s, ((it >> 1) & 1) ^ 1, abort_flag);
      if (ok) {
        const int col = p.col0 + min(tn * BN + t, p.N - 1);
        const int16_t* xb = p.act.bsums + (int64_t)col * p.act.col_stride_bs;
        const float* xd = p.act.d + (int64_t)col * p.act.col_stride_d;
        uint8_t* st = smem + s * kStageBytes;
        // activations: this warp's 32 columns, 8 columns x 4 chunks (64 contiguous bytes each) per instruction
        {
          const int col8 = lane & 7, cq = lane >> 3;
          const uint32_t bbase = smem_u32(st + kOffB);
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            const int cl = 32 * warp + 8 * g + col8;                       // column within the tile
            const int8_t* src = p.act.qs + (int64_t)(p.col0 + min(tn * BN + cl, p.N - 1)) * p.act.col_stride_qs + kb * QK_K;
            const uint32_t dst = bbase + (uint32_t)(cl >> 3) * kGroupStride + (uint32_t)(cl & 7) * 16;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const int c = 4 * i + cq;
              asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + c * kChunkStride), "l"(src + 16 * c) : "memory");
            }
          }
        }
        {
          const int4* bs = reinterpret_cast<const int4*>(xb + kb * 16);
          const int4 b0 = __ldg(bs), b1 = __ldg(bs + 1);
          const int w[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
          uint32_t ps[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) ps[j] = (uint32_t)((int)(short)(w[j] & 0xffff) + (w[j] >> 16)) & 0xffffu;
          *reinterpret_cast<uint4*>(st + kOffColMeta + t * 16) =
              make_uint4(ps[0] | (ps[1] << 16), ps[2] | (ps[3] << 16), ps[4] | (ps[5] << 16), ps[6] | (ps[7] << 16));
          *reinterpret_cast<float*>(st + kOffDx + t * 4) = __ldg(xd + kb);
        }
        // weights of row t: scales, then the two int8 operands
        const uint4 h = blk[0];
        const uint32_t s0 = h.y, s1 = h.z, s2 = h.w;
        const uint32_t sc_lo4 = s0 & 0x3f3f3f3fu, mn_lo4 = s1 & 0x3f3f3f3fu;
        const uint32_t sc_hi4 = (s2 & 0x0f0f0f0fu) | (((s0 >> 6) & 0x03030303u) << 4);
        const uint32_t mn_hi4 = ((s2 >> 4) & 0x0f0f0f0fu) | (((s1 >> 6) & 0x03030303u) << 4);
        *reinterpret_cast<uint4*>(st + kOffRowMeta + t * 16) =
            make_uint4(__float_as_uint(h2f((uint16_t)(h.x & 0xffffu))), __float_as_uint(h2f((uint16_t)(h.x >> 16))), mn_lo4, mn_hi4);
        uint8_t* alo = st + kOffAlo + core_off;
        uint8_t* ahi = st + kOffAhi + core_off;
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          const uint4 v0 = blk[1 + 2 * g], v1 = blk[2 + 2 * g];
          const uint32_t scw = g < 2 ? sc_lo4 : sc_hi4;
          const uint32_t sca = (scw >> (16 * (g & 1))) & 0xffu, scb = (scw >> (16 * (g & 1) + 8)) & 0xffu;
          const uint32_t la = sca & 7u, ha = sca >> 3, lb = scb & 7u, hb = scb >> 3;
          const uint32_t q[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
          uint32_t lo[8], hi[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) { lo[i] = q[i] & 0x0f0f0f0fu; hi[i] = (q[i] >> 4) & 0x0f0f0f0fu; }
          // sub-block 2g (low nibbles): chunks 4g, 4g+1; sub-block 2g+1 (high nibbles): chunks 4g+2, 4g+3
          *reinterpret_cast<uint4*>(alo + (4 * g + 0) * kChunkStride) = make_uint4(lo[0] * la, lo[1] * la, lo[2] * la, lo[3] * la);
          *reinterpret_cast<uint4*>(alo + (4 * g + 1) * kChunkStride) = make_uint4(lo[4] * la, lo[5] * la, lo[6] * la, lo[7] * la);
          *reinterpret_cast<uint4*>(alo + (4 * g + 2) * kChunkStride) = make_uint4(hi[0] * lb, hi[1] * lb, hi[2] * lb, hi[3] * lb);
          *reinterpret_cast<uint4*>(alo + (4 * g + 3) * kChunkStride) = make_uint4(hi[4] * lb, hi[5] * lb, hi[6] * lb, hi[7] * lb);
          *reinterpret_cast<uint4*>(ahi + (4 * g + 0) * kChunkStride) = make_uint4(lo[0] * ha, lo[1] * ha, lo[2] * ha, lo[3] * ha);
          *reinterpret_cast<uint4*>(ahi + (4 * g + 1) * kChunkStride) = make_uint4(lo[4] * ha, lo[5] * ha, lo[6] * ha, lo[7] * ha);
          *reinterpret_cast<uint4*>(ahi + (4 * g + 2) * kChunkStride) = make_uint4(hi[0] * hb, hi[1] * hb, hi[2] * hb, hi[3] * hb);
          *reinterpret_cast<uint4*>(ahi + (4 * g + 3) * kChunkStride) = make_uint4(hi[4] * hb, hi[5] * hb, hi[6] * hb, hi[7] * hb);
        }
        asm volatile("cp.async.wait_all;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic-proxy writes -> visible to the tensor core's reads
        mbar_arrive(full + s);
      }
      tile = ntile;
      kb = nkbi;
    }
    if (*abort_flag) {
      // a raw copy may still be in flight: give it a bounded moment before the CTA's shared memory goes away
      for (int spins = 0; spins < (1 << 16) && !mbar_try_wait(raw_full, it & 1); ++spins) {}
    }
  } else if (warp == kMmaWarp) {
    // ---------------------------------------------------------------- MMA issue (one thread)
    if (lane == 0) {
      int it = 0, last_commit = -1;
      bool live = true;
      for (int tile = blockIdx.x; live && tile < ntiles; tile += gridDim.x) {
        for (int kb = 0; kb < nkb; ++kb, ++it) {
          const int s = it & 1;
          if (!mbar_wait(full + s, (it >> 1) & 1, abort_flag)) { live = false; break; }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          uint8_t* st = smem + s * kStageBytes;
          const uint32_t a_lo = smem_u32(st + kOffAlo), a_hi = smem_u32(st + kOffAhi), b = smem_u32(st + kOffB);
          const uint32_t d_lo = tmem_base + (uint32_t)s * 256u, d_hi = d_lo + 128u;
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const uint64_t db = operand_desc(b + 2 * j * kChunkStride);
            mma_i8(d_lo, operand_desc(a_lo + 2 * j * kChunkStride), db, j > 0 ? 1u : 0u);
            mma_i8(d_hi, operand_desc(a_hi + 2 * j * kChunkStride), db, j > 0 ? 1u : 0u);
          }
          mma_commit(tmem_full + s);
          last_commit = it;
        }
      }
      if (!live && last_commit >= 0) {
        // gave up: let the tensor core finish what was issued before the TMEM goes away (bounded)
        uint64_t* bar = tmem_full + (last_commit & 1);
        const uint32_t parity = (last_commit >> 1) & 1;
        for (int spins = 0; spins < (1 << 20) && !mbar_try_wait(bar, parity); ++spins) {}
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue
    const int quarter = warp & 3;                       // the TMEM lanes this warp may read: 32*quarter ..
    const int cgroup = (warp - kEpilogueWarp0) >> 2;    // columns 32*cgroup .. 32*cgroup+31
    const int r = 32 * quarter + lane;                  // row of the tile = TMEM lane
    const uint32_t lane_addr = tmem_base + ((uint32_t)(32 * quarter) << 16) + (uint32_t)(32 * cgroup);
    int it = 0;
    bool live = true;
    for (int tile = blockIdx.x; live && tile < ntiles; tile += gridDim.x) {
      const int tm = tile / nt, tn = tile - tm * nt;
      float acc[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) acc[i] = 0.0f;
      for (int kb = 0; kb < nkb; ++kb, ++it) {
        const int s = it & 1;
        if (!mbar_wait(tmem_full + s, (it >> 1) & 1, abort_flag)) { live = false; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint8_t* st = smem + s * kStageBytes;
        const uint4 rm = *reinterpret_cast<const uint4*>(st + kOffRowMeta + r * 16);
        const float d = __uint_as_float(rm.x), dmin = __uint_as_float(rm.y);
        const int mn_lo4 = (int)rm.z, mn_hi4 = (int)rm.w;
#pragma unroll
        for (int c8 = 0; c8 < 4; ++c8) {
          uint32_t lo[8], hi[8];
          tmem_ld8(lane_addr + (uint32_t)s * 256u + (uint32_t)(8 * c8), lo);
          tmem_ld8(lane_addr + (uint32_t)s * 256u + 128u + (uint32_t)(8 * c8), hi);
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int col = 32 * cgroup + 8 * c8 + i;
            const uint4 cm = *reinterpret_cast<const uint4*>(st + kOffColMeta + col * 16);
            const float dx = *reinterpret_cast<const float*>(st + kOffDx + col * 4);
            const int isum = (int)lo[i] + 8 * (int)hi[i];
            int msum = __dp2a_lo((int)cm.x, mn_lo4, 0);
            msum = __dp2a_hi((int)cm.y, mn_lo4, msum);
            msum = __dp2a_lo((int)cm.z, mn_hi4, msum);
            msum = __dp2a_hi((int)cm.w, mn_hi4, msum);
            const float d_all = __fmul_rn(dx, d), d_min = __fmul_rn(dx, dmin);
            const float bv = __fmaf_rn(d_all, (float)isum, -__fmul_rn(d_min, (float)msum));
            acc[8 * c8 + i] = __fadd_rn(acc[8 * c8 + i], bv);
          }
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive(epi_done + s);
      }
      if (!live) break;
      const int row = tm * BM + r;
      if (row < p.M) {
        float* yr = p.y + (size_t)row * p.ldy + p.col0;
        const int c0 = tn * BN + 32 * cgroup;
#pragma unroll
        for (int i = 0; i < 32; ++i)
          if (c0 + i < p.N) yr[c0 + i] = acc[i];
      }
    }
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag && p.status) atomicExch(p.status, 1);
  if (warp == kMmaWarp) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
  }
}

}  // namespace

bool gemm_tc_supported(int type, int K, int ncols, const void* W, int64_t row_bytes, const ActPlanes& act) {
  return type == T_Q4_K && ncols >= kGemmTcMinCols && K % QK_K == 0 && (reinterpret_cast<uintptr_t>(W) & 15) == 0 && row_bytes % 16 == 0 &&
         act.bsums != nullptr && (reinterpret_cast<uintptr_t>(act.qs) & 15) == 0 && act.col_stride_qs % 16 == 0 &&
         (reinterpret_cast<uintptr_t>(act.bsums) & 15) == 0 && act.col_stride_bs % 8 == 0;
}

cudaError_t launch_gemm_q4k_tc(const GemvArgs& a, int ncols, int sm_count, cudaStream_t st) {
  static unsigned configured = 0;  // one bit per device
  int dev = 0;
  cudaGetDevice(&dev);
  if (!(configured & (1u << (dev & 31)))) {
    const cudaError_t e = cudaFuncSetAttribute(gemm_q4k_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (e != cudaSuccess) return e;
    configured |= 1u << (dev & 31);
  }
  GemmArgs g{};
  g.W = a.W;
  g.row_bytes = a.row_bytes;
  g.M = a.M;
  g.K = a.K;
  g.N = ncols;
  g.act = a.act;
  g.col0 = a.col0;
  g.y = a.y;
  g.ldy = a.ldy;
  g.status = a.status;
  const int tiles = ((a.M + BM - 1) / BM) * ((ncols + BN - 1) / BN);
  const int grid = tiles < sm_count ? tiles : sm_count;
  gemm_q4k_tc_kernel<<<grid, kThreads, kSmemBytes, st>>>(g);
  return cudaGetLastError();
}

}  // namespace emelb
