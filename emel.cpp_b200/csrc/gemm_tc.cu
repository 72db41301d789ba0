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
//   * one MMA has K = 32 = one sub-block.  The activations are the M operand (128
//     tokens = TMEM lanes) and the two weight operands sit side by side in the N
//     operand (128 rows of q*lo, then 128 rows of q*hi), so ONE 128 x 256 x 32 MMA
//     per sub-block produces both D_lo (columns 0-127) and D_hi (128-255) and the
//     activation slice is fetched from shared memory once; 8 MMAs cover a
//     super-block of 256; then the accumulators are read back (tcgen05.ld) and
//     folded into f32 registers with the block's scales — the float chain stays on
//     the CUDA cores because its order and roundings are part of the contract.
//
// CTA = 128 rows x 128 columns, 21 warps:
//   warps 0-3   producers: the 128 GGUF blocks of a super-block column are staged
//               raw (16-byte cp.async, coalesced along rows) one iteration ahead;
//               thread p expands row p into the two int8 operands in the
//               canonical no-swizzle K-major layout (8 rows x 16 bytes core
//               matrices).  The activation tile comes by bulk copy: a small
//               pre-pass has already laid it out in that same layout (one
//               contiguous 32 KB slab + per-column block sums and scales per
//               128 columns x 256 K)
//   warp  4     allocates TMEM, issues the MMAs, commits to two mbarriers
//   warps 5-20  epilogue: four warps per TMEM lane quarter, 32 columns each; msum
//               on the legacy mma.sync path in the accumulator-fragment layout
//   warp  21    one thread starts the bulk copies of the next activation tile the
//               moment an operand stage is released
// Two operand stages are released by the MMA's completion, two TMEM accumulator
// pairs and four small per-block scale slots by the epilogue, so producers,
// tensor cores and epilogue work on different super-blocks at once.
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
constexpr int kLoaderWarp = 21;
constexpr int kThreads = 22 * 32;
constexpr int kEpilogueWarps = 16;
constexpr int kStages = 2;

// shared memory map (bytes)
constexpr int kOperandBytes = BM * 256;                 // one int8 operand tile of a super-block: 32 KB
constexpr int kChunkStride = (BM / 8) * 128;            // activation tile: next 16-byte K chunk of the 128 tokens (2048 B)
constexpr int kChunkStrideW = 2 * kChunkStride;         // weight tile: 256 operand rows (q*lo, then q*hi) per chunk (4096 B)
constexpr int kGroupStride = 128;                       // next 8-row core matrix (stride byte offset)
constexpr int kStageBytes = 3 * kOperandBytes;          // weights (q*lo | q*hi interleaved per K chunk: 64 KB), activations
constexpr int kOffW = 0, kOffX = 2 * kOperandBytes;
constexpr int kMetaSlots = 4;
constexpr int kColMetaBytes = BN * 16 + BN * 4;         // per column: 8 pair sums as int8 low/high parts, then the scales dx
constexpr int kRowMetaBytes = 12;                       // per row: {d, dmin} as f16 bits, mins[8]
constexpr int kMetaBytes = BM * kRowMetaBytes + kColMetaBytes;
constexpr int kOffRowMeta = 0, kOffColMeta = BM * kRowMetaBytes, kOffDx = kOffColMeta + BN * 16;
constexpr int kRawBytes = BM * Q4_K_BYTES;              // raw GGUF blocks of one super-block column: 18,432 B
constexpr int kBarBytes = 128;                          // full[2], mma_done[2], tmem_full[2], epi_done[2], tmem base, abort
constexpr int kSmemBytes = kStages * kStageBytes + kMetaSlots * kMetaBytes + kRawBytes + kBarBytes + 128;  // + alignment slack
// the activation tile a pre-pass writes for (128 columns, one super-block): operand B, then the column meta
constexpr int kTileBytes = kOperandBytes + kColMetaBytes;

constexpr int kWaitSpins = 1 << 22;
constexpr uint32_t kSuspendHintNs = 10000;
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
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"   // may sleep up to the hint instead of spinning
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity), "r"(kSuspendHintNs)
      : "memory");
  return ok != 0;
}

// bounded wait; false when it gave up or another role already raised the abort flag
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  unsigned long long t0 = 0;
  for (int spins = 0; spins < kWaitSpins; ++spins) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((spins & 15) == 15) {
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

__device__ __forceinline__ uint64_t operand_desc(uint32_t saddr, uint32_t chunk_stride) {
  // K-major, no swizzle: 14-bit fields in 16-byte units; descriptor version 1 (sm_100)
  uint64_t d = 0;
  d |= (uint64_t)((saddr >> 4) & 0x3fffu);
  d |= (uint64_t)((chunk_stride >> 4) & 0x3fffu) << 16;   // leading byte offset: between the two 16-byte K chunks
  d |= (uint64_t)((kGroupStride >> 4) & 0x3fffu) << 32;   // stride byte offset: between 8-row groups
  d |= (uint64_t)1 << 46;
  return d;
}

// instruction descriptor: D = s32, A = B = signed 8-bit, both K-major, M = 128 tokens, N = 256 weight-operand rows
constexpr uint32_t kInstrDesc = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)((2 * BM) >> 3) << 17) | ((uint32_t)(BN >> 4) << 24);

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

// 16 TMEM lanes x 16 columns in the m16n8 accumulator-fragment layout: v[0..3] = columns 0-7, v[4..7] = columns
// 8-15; within a block thread (g, t) gets (row g, col 2t), (row g, col 2t+1), (row g+8, col 2t), (row g+8, col 2t+1)
__device__ __forceinline__ void tmem_ld_16x256b_x2(uint32_t taddr, uint32_t (&v)[8]) {
  asm volatile("tcgen05.ld.sync.aligned.16x256b.x2.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7])
               : "r"(taddr)
               : "memory");
}

// D(16 tokens x 8 weight rows, f32) = A(16x16, f16) * B(16x8, f16) with A[token][k] = low parts (k < 8) and
// 128 * high parts (k >= 8) of the token's block sums (a_lo0/a_lo1, a_hi0/a_hi1: tokens g, g+8) and
// B[k][row] = B[k+8][row] = the weight row's k-th min
__device__ __forceinline__ void mma_m16n8k16_f16(float (&dd)[4], uint32_t a_lo0, uint32_t a_lo1, uint32_t a_hi0, uint32_t a_hi1,
                                                 uint32_t b_mins) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
      : "=f"(dd[0]), "=f"(dd[1]), "=f"(dd[2]), "=f"(dd[3])
      : "r"(a_lo0), "r"(a_lo1), "r"(a_hi0), "r"(a_hi1), "r"(b_mins), "r"(b_mins), "f"(0.0f), "f"(0.0f), "f"(0.0f), "f"(0.0f));
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
  const uint8_t* tiles;   // [ceil(N/128)][K/256][kTileBytes]
  float* y;
  int64_t ldy;
  int* status;
};

// pre-pass: the quantized activation planes of columns col0.. -> tiles in operand order.
// grid (K/256, ceil(N/128)), 256 threads; columns past N are zero.
__global__ void __launch_bounds__(256) tile_activations_kernel(ActPlanes act, int col0, int N, int K, uint8_t* tiles) {
  const int kb = blockIdx.x, tn = blockIdx.y, nkb = K / QK_K;
  uint8_t* tile = tiles + ((size_t)tn * nkb + kb) * kTileBytes;
  for (int q = threadIdx.x; q < BN * 16; q += 256) {
    const int col = q & (BN - 1), c = q >> 7;           // piece q = (chunk c, column col) lands at q*16
    const int gc = tn * BN + col;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (gc < N) v = *reinterpret_cast<const uint4*>(act.qs + (int64_t)(col0 + gc) * act.col_stride_qs + kb * QK_K + 16 * c);
    *reinterpret_cast<uint4*>(tile + (size_t)q * 16) = v;
  }
  if (threadIdx.x < BN) {
    const int col = threadIdx.x, gc = tn * BN + col;
    uint4 cm = make_uint4(0, 0, 0, 0);
    float dx = 0.0f;
    if (gc < N) {
      const int4* bs = reinterpret_cast<const int4*>(act.bsums + (int64_t)(col0 + gc) * act.col_stride_bs + kb * 16);
      const int4 b0 = bs[0], b1 = bs[1];
      const int w[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
      // pair sums (|s| <= 4064) split as s = 128*hi + lo with 0 <= lo < 128, so both parts are int8 for dp4a
      uint32_t bl[8], bh[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int sj = (int)(short)(w[j] & 0xffff) + (w[j] >> 16);
        bl[j] = (uint32_t)(sj & 127);
        bh[j] = (uint32_t)(sj >> 7) & 0xffu;
      }
      cm = make_uint4(bl[0] | (bl[1] << 8) | (bl[2] << 16) | (bl[3] << 24), bl[4] | (bl[5] << 8) | (bl[6] << 16) | (bl[7] << 24),
                      bh[0] | (bh[1] << 8) | (bh[2] << 16) | (bh[3] << 24), bh[4] | (bh[5] << 8) | (bh[6] << 16) | (bh[7] << 24));
      dx = act.d[(int64_t)(col0 + gc) * act.col_stride_d + kb];
    }
    *reinterpret_cast<uint4*>(tile + kOperandBytes + col * 16) = cm;
    *reinterpret_cast<float*>(tile + kOperandBytes + BN * 16 + col * 4) = dx;
  }
}

__global__ void __launch_bounds__(kThreads, 1) gemm_q4k_tc_kernel(const GemmArgs p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
  uint8_t* meta = smem + kStages * kStageBytes;
  uint8_t* raw = meta + kMetaSlots * kMetaBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(raw + kRawBytes);
  uint64_t* full = bars;            // [2] producers + bulk copies -> MMA: operands of a super-block are in shared memory
  uint64_t* mma_done = bars + 2;    // [2] MMA -> producers: the operand stage may be overwritten
  uint64_t* tmem_full = bars + 4;   // [2] MMA -> epilogue: the accumulator pair holds a finished super-block
  uint64_t* epi_done = bars + 6;    // [2] epilogue -> MMA (accumulator pair free) and producers (scale slot free)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(full + s, kProducerThreads + 1);
      mbar_init(mma_done + s, 1);
      mbar_init(tmem_full + s, 1);
      mbar_init(epi_done + s, kEpilogueWarps);
    }
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
    const int t = threadIdx.x;  // row t of the weight tile
    const uint32_t core_off = (uint32_t)(t >> 3) * kGroupStride + (uint32_t)(t & 7) * 16;
    // raw staging of iteration (tile, kb): 1152 16-byte pieces, piece g = (row g/9, part g%9) lands at g*16
    auto issue_raw = [&](int tile, int kb) {
      const int tm = tile / nt;
      const uint32_t rbase = smem_u32(raw);
#pragma unroll
      for (int j = 0; j < 9; ++j) {
        const int g = t + 128 * j;
        const int rr = g / 9, part = g - 9 * rr;
        const int row = min(tm * BM + rr, p.M - 1);           // rows past M repeat the last one; never stored
        const uint8_t* src = p.W + (size_t)row * p.row_bytes + (size_t)kb * Q4_K_BYTES + 16 * part;
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(rbase + 16u * (uint32_t)g), "l"(src) : "memory");
      }
      asm volatile("cp.async.commit_group;" ::: "memory");
    };
    // One flat loop over (tile, super-block).  The 128 producers meet at named barriers every
    // iteration, so nobody leaves early: a wait that gave up only skips work, and the loop ends
    // for everyone at the abort check right after a barrier.
    int it = 0, tile = blockIdx.x, kb = 0;
    if (tile < ntiles) issue_raw(tile, 0);
    for (; tile < ntiles; ++it) {
      const int tn = tile % nt;
      const int s = it & 1, m = it & (kMetaSlots - 1);
      asm volatile("cp.async.wait_group 0;" ::: "memory");
      asm volatile("bar.sync 1, 128;" ::: "memory");          // everybody's pieces of this iteration's raw blocks landed
      uint4 blk[9];
#pragma unroll
      for (int i = 0; i < 9; ++i) blk[i] = *reinterpret_cast<const uint4*>(raw + t * Q4_K_BYTES + 16 * i);
      asm volatile("bar.sync 1, 128;" ::: "memory");          // everybody has read: the staging buffer is free
      if (*abort_flag) break;
      int ntile = tile, nkbi = kb + 1;
      if (nkbi == nkb) { nkbi = 0; ntile += gridDim.x; }
      if (ntile < ntiles) issue_raw(ntile, nkbi);
      // operand stage s was consumed by the MMAs of iteration it-2; those were issued after the epilogue of
      // it-4 had finished, which is the last reader of scale slot m
      const bool ok = mbar_wait(mma_done + s, ((it >> 1) & 1) ^ 1, abort_flag);
      if (ok) {
        uint8_t* st = smem + s * kStageBytes;
        uint8_t* mt_ = meta + m * kMetaBytes;
        // weights of row t: scales, then the two int8 operands
        const uint4 h = blk[0];
        const uint32_t s0 = h.y, s1 = h.z, s2 = h.w;
        const uint32_t sc_lo4 = s0 & 0x3f3f3f3fu, mn_lo4 = s1 & 0x3f3f3f3fu;
        const uint32_t sc_hi4 = (s2 & 0x0f0f0f0fu) | (((s0 >> 6) & 0x03030303u) << 4);
        const uint32_t mn_hi4 = ((s2 >> 4) & 0x0f0f0f0fu) | (((s1 >> 6) & 0x03030303u) << 4);
        {
          uint32_t* rmw = reinterpret_cast<uint32_t*>(mt_ + kOffRowMeta + t * kRowMetaBytes);
          rmw[0] = h.x;
          rmw[1] = mn_lo4;
          rmw[2] = mn_hi4;
        }
        uint8_t* alo = st + kOffW + core_off;                  // operand rows 0-127: q*lo
        uint8_t* ahi = alo + kChunkStride;                     // operand rows 128-255: q*hi (16 core-matrix groups further)
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
          *reinterpret_cast<uint4*>(alo + (4 * g + 0) * kChunkStrideW) = make_uint4(lo[0] * la, lo[1] * la, lo[2] * la, lo[3] * la);
          *reinterpret_cast<uint4*>(alo + (4 * g + 1) * kChunkStrideW) = make_uint4(lo[4] * la, lo[5] * la, lo[6] * la, lo[7] * la);
          *reinterpret_cast<uint4*>(alo + (4 * g + 2) * kChunkStrideW) = make_uint4(hi[0] * lb, hi[1] * lb, hi[2] * lb, hi[3] * lb);
          *reinterpret_cast<uint4*>(alo + (4 * g + 3) * kChunkStrideW) = make_uint4(hi[4] * lb, hi[5] * lb, hi[6] * lb, hi[7] * lb);
          *reinterpret_cast<uint4*>(ahi + (4 * g + 0) * kChunkStrideW) = make_uint4(lo[0] * ha, lo[1] * ha, lo[2] * ha, lo[3] * ha);
          *reinterpret_cast<uint4*>(ahi + (4 * g + 1) * kChunkStrideW) = make_uint4(lo[4] * ha, lo[5] * ha, lo[6] * ha, lo[7] * ha);
          *reinterpret_cast<uint4*>(ahi + (4 * g + 2) * kChunkStrideW) = make_uint4(hi[0] * hb, hi[1] * hb, hi[2] * hb, hi[3] * hb);
          *reinterpret_cast<uint4*>(ahi + (4 * g + 3) * kChunkStrideW) = make_uint4(hi[4] * hb, hi[5] * hb, hi[6] * hb, hi[7] * hb);
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic-proxy writes -> visible to the tensor core's reads
        mbar_arrive(full + s);
      }
      tile = ntile;
      kb = nkbi;
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
  } else if (warp == kMmaWarp) {
    // ---------------------------------------------------------------- MMA issue (one thread)
    if (lane == 0) {
      int it = 0, last_commit = -1;
      bool live = true;
      for (int tile = blockIdx.x; live && tile < ntiles; tile += gridDim.x) {
        for (int kb = 0; kb < nkb; ++kb, ++it) {
          const int s = it & 1;
          // operands in place, and the accumulator pair drained by the epilogue of iteration it-2
          if (!mbar_wait(full + s, (it >> 1) & 1, abort_flag)) { live = false; break; }
          if (!mbar_wait(epi_done + s, ((it >> 1) & 1) ^ 1, abort_flag)) { live = false; break; }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          uint8_t* st = smem + s * kStageBytes;
          const uint32_t xop = smem_u32(st + kOffX), wop = smem_u32(st + kOffW);
          const uint32_t d_acc = tmem_base + (uint32_t)s * 256u;   // columns 0-127: D_lo, 128-255: D_hi
#pragma unroll
          for (int j = 0; j < 8; ++j)
            mma_i8(d_acc, operand_desc(xop + 2 * j * kChunkStride, kChunkStride), operand_desc(wop + 2 * j * kChunkStrideW, kChunkStrideW),
                   j > 0 ? 1u : 0u);
          mma_commit(mma_done + s);
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
  } else if (warp == kLoaderWarp) {
    // ---------------------------------------------------------------- activation tile loader (one thread)
    if (lane == 0) {
      int it = 0;
      bool live = true;
      for (int tile = blockIdx.x; live && tile < ntiles; tile += gridDim.x) {
        const int tn = tile % nt;
        for (int kb = 0; kb < nkb; ++kb, ++it) {
          const int s = it & 1;
          if (!mbar_wait(mma_done + s, ((it >> 1) & 1) ^ 1, abort_flag)) { live = false; break; }
          uint8_t* st = smem + s * kStageBytes;
          uint8_t* mt_ = meta + (it & (kMetaSlots - 1)) * kMetaBytes;
          const uint8_t* tile_src = p.tiles + ((size_t)tn * nkb + kb) * kTileBytes;
          mbar_arrive_expect_tx(full + s, kTileBytes);
#pragma unroll
          for (int q = 0; q < 4; ++q)
            bulk_g2s(st + kOffX + q * (kOperandBytes / 4), tile_src + q * (kOperandBytes / 4), kOperandBytes / 4, full + s);
          bulk_g2s(mt_ + kOffColMeta, tile_src + kOperandBytes, kColMetaBytes, full + s);
          // the tile this stage gets next (two super-blocks ahead, same tile row while kb + 2 < nkb) towards L2:
          // the copy above is issued only when the stage frees up, so its latency is on the critical path
          if (kb + 2 < nkb)
            asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(tile_src + 2 * (size_t)kTileBytes), "r"(kTileBytes) : "memory");
        }
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue
    // TMEM lanes are tokens, TMEM columns weight rows.  The warp owns 32 tokens (its lane quarter) x 32 weight
    // rows.  Accumulators are read in the 16x256b shape, whose register layout is the m16n8 C fragment: thread
    // (g = lane/4, t = lane%4) holds tokens g and g+8, weight rows 2t and 2t+1 of every 8-row block.
    // msum = sum_j bsum_j * m_j for the same elements comes from one legacy-path mma.sync per (16 tokens x 8
    // weight rows): A = the token's block sums split as lo + 128*hi, B = the weight row's 8 mins (twice), so
    // every f16 operand and every f32 partial sum is an exact integer.
    const int quarter = warp & 3;                       // the TMEM lanes this warp may read: tokens 32*quarter ..
    const int cgroup = (warp - kEpilogueWarp0) >> 2;    // weight rows 32*cgroup .. 32*cgroup+31
    const int g = lane >> 2, t = lane & 3;
    int it = 0;
    bool live = true;
    for (int tile = blockIdx.x; live && tile < ntiles; tile += gridDim.x) {
      const int tm = tile / nt, tn = tile - tm * nt;
      float acc[4][4][2];   // [token g + 8*j][8-row block][weight row 2t + e]
#pragma unroll
      for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int nb = 0; nb < 4; ++nb) acc[j][nb][0] = acc[j][nb][1] = 0.0f;
      for (int kb = 0; kb < nkb; ++kb, ++it) {
        const int s = it & 1;
        if (!mbar_wait(tmem_full + s, (it >> 1) & 1, abort_flag)) { live = false; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint8_t* mt_ = meta + (it & (kMetaSlots - 1)) * kMetaBytes;
        const uint8_t* tokmeta = mt_ + kOffColMeta + (32 * quarter) * 16;                       // per token: 8 lo, 8 hi parts
        const float* dxs = reinterpret_cast<const float*>(mt_ + kOffDx) + 32 * quarter;          // per token: dx
        const uint8_t* wmeta = mt_ + kOffRowMeta + (32 * cgroup) * kRowMetaBytes;                // per weight row: {d, dmin}, mins
        // B fragments of the four 8-row blocks: weight row g of the block, mins 2t and 2t+1
        uint32_t bfm[4];
#pragma unroll
        for (int nb = 0; nb < 4; ++nb) {
          const uint32_t m2 = *reinterpret_cast<const uint16_t*>(wmeta + (8 * nb + g) * kRowMetaBytes + 4 + 2 * t);
          const __half2 fm = __halves2half2(__ushort2half_rn((unsigned short)(m2 & 0xffu)), __ushort2half_rn((unsigned short)(m2 >> 8)));
          bfm[nb] = *reinterpret_cast<const uint32_t*>(&fm);
        }
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          // tokens g + 16*hh and g + 8 + 16*hh: scale and the A fragments (block sums 2t, 2t+1: low parts, high parts)
          float dx[2];
          uint32_t afl[2], afh[2];
#pragma unroll
          for (int rr = 0; rr < 2; ++rr) {
            const int tok = 16 * hh + 8 * rr + g;
            dx[rr] = dxs[tok];
            const uint32_t l2 = *reinterpret_cast<const uint16_t*>(tokmeta + tok * 16 + 2 * t);
            const uint32_t h2 = *reinterpret_cast<const uint16_t*>(tokmeta + tok * 16 + 8 + 2 * t);
            const __half2 fl = __halves2half2(__ushort2half_rn((unsigned short)(l2 & 0xffu)), __ushort2half_rn((unsigned short)(l2 >> 8)));
            const __half2 fh = __halves2half2(__short2half_rn((short)((int)(int8_t)(h2 & 0xffu) * 128)),
                                              __short2half_rn((short)((int)(int8_t)(h2 >> 8) * 128)));
            afl[rr] = *reinterpret_cast<const uint32_t*>(&fl);
            afh[rr] = *reinterpret_cast<const uint32_t*>(&fh);
          }
          const uint32_t tbase = tmem_base + ((uint32_t)(32 * quarter + 16 * hh) << 16) + (uint32_t)s * 256u + (uint32_t)(32 * cgroup);
#pragma unroll
          for (int cp = 0; cp < 2; ++cp) {
            uint32_t lo[8], hi[8];
            tmem_ld_16x256b_x2(tbase + (uint32_t)(16 * cp), lo);
            tmem_ld_16x256b_x2(tbase + 128u + (uint32_t)(16 * cp), hi);
            float ms[2][4];
#pragma unroll
            for (int q2 = 0; q2 < 2; ++q2) mma_m16n8k16_f16(ms[q2], afl[0], afl[1], afh[0], afh[1], bfm[2 * cp + q2]);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
            for (int q2 = 0; q2 < 2; ++q2) {
              const int nb = 2 * cp + q2;
              const uint8_t* wm = wmeta + (8 * nb + 2 * t) * kRowMetaBytes;
              const uint32_t db0 = *reinterpret_cast<const uint32_t*>(wm), db1 = *reinterpret_cast<const uint32_t*>(wm + kRowMetaBytes);
              const float dw[2] = {h2f((uint16_t)(db0 & 0xffffu)), h2f((uint16_t)(db1 & 0xffffu))};
              const float dminw[2] = {h2f((uint16_t)(db0 >> 16)), h2f((uint16_t)(db1 >> 16))};
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const int rr = e >> 1, ce = e & 1;
                const int isum = (int)lo[4 * q2 + e] + 8 * (int)hi[4 * q2 + e];
                const float d_all = __fmul_rn(dx[rr], dw[ce]), d_min = __fmul_rn(dx[rr], dminw[ce]);
                const float bv = __fmaf_rn(d_all, (float)isum, -__fmul_rn(d_min, ms[q2][e]));
                acc[2 * hh + rr][nb][ce] = __fadd_rn(acc[2 * hh + rr][nb][ce], bv);
              }
            }
          }
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive(epi_done + s);
      }
      if (!live) break;
#pragma unroll
      for (int nb = 0; nb < 4; ++nb)
#pragma unroll
        for (int ce = 0; ce < 2; ++ce) {
          const int row = tm * BM + 32 * cgroup + 8 * nb + 2 * t + ce;      // weight row
          if (row < p.M) {
            float* yr = p.y + (size_t)row * p.ldy + tn * BN + 32 * quarter + g;
#pragma unroll
            for (int j = 0; j < 4; ++j)
              if (tn * BN + 32 * quarter + 8 * j + g < p.N) yr[8 * j] = acc[j][nb][ce];
          }
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

size_t gemm_tc_workspace_bytes(int K, int ncols) {
  return (size_t)((ncols + BN - 1) / BN) * (size_t)(K / QK_K) * kTileBytes;
}

bool gemm_tc_supported(int type, int K, int ncols, const void* W, int64_t row_bytes, const ActPlanes& act) {
  return type == T_Q4_K && ncols >= kGemmTcMinCols && K % QK_K == 0 && (reinterpret_cast<uintptr_t>(W) & 15) == 0 && row_bytes % 16 == 0 &&
         act.bsums != nullptr && (reinterpret_cast<uintptr_t>(act.qs) & 15) == 0 && act.col_stride_qs % 16 == 0 &&
         (reinterpret_cast<uintptr_t>(act.bsums) & 15) == 0 && act.col_stride_bs % 8 == 0;
}

// two launches: the activation tiling pre-pass (into `workspace`, gemm_tc_workspace_bytes) and the product
cudaError_t launch_gemm_q4k_tc(const GemvArgs& a, int ncols, int sm_count, uint8_t* workspace, cudaStream_t st) {
  // per host thread (one context, one lane per thread): no shared mutable state between lanes
  static thread_local unsigned configured = 0;  // one bit per device
  int dev = 0;
  cudaGetDevice(&dev);
  if (!(configured & (1u << (dev & 31)))) {
    const cudaError_t e = cudaFuncSetAttribute(gemm_q4k_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (e != cudaSuccess) return e;
    configured |= 1u << (dev & 31);
  }
  const int nt = (ncols + BN - 1) / BN;
  cudaError_t e = cudaSuccess;
  if (!a.tc_ws_reuse) {  // else the workspace still holds these planes in operand order (same K, columns, col0)
    tile_activations_kernel<<<dim3(a.K / QK_K, nt), 256, 0, st>>>(a.act, a.col0, ncols, a.K, workspace);
    e = cudaGetLastError();
    if (e != cudaSuccess) return e;
  }
  GemmArgs g{};
  g.W = a.W;
  g.row_bytes = a.row_bytes;
  g.M = a.M;
  g.K = a.K;
  g.N = ncols;
  g.tiles = workspace;
  g.y = a.y + a.col0;
  g.ldy = a.ldy;
  g.status = a.status;
  const int tiles = ((a.M + BM - 1) / BM) * nt;
  const int grid = tiles < sm_count ? tiles : sm_count;
  gemm_q4k_tc_kernel<<<grid, kThreads, kSmemBytes, st>>>(g);
  return cudaGetLastError();
}

}  // namespace emelb
