// 5 to 31 columns of Q4_K weights x Q8_K activations (a decode step of several sequences): too many columns for
// the CUDA-core mat-vec kernels, whose integer dot products per weight byte grow with the column count, and too
// few to fill the 128-token tile of the tcgen05 kernel.  The integer part runs on the legacy tensor path,
// mma.sync.m16n8k32 (s8 x s8 -> s32): one instruction = one 32-weight sub-block of 16 rows against 8 columns.
//
// Per 256-weight super-block and (row, column) the value is the reference's
//   fma(d*dx, isum, -(dmin*dx)*msum),  isum = sum_j sc_j * dot_j(q, x),  msum = sum_j m_j * bsum_j
// (src/emel/kernel/x86_64/actions.hpp:859-866) added to the row sum in ascending block order: dot_j comes out of
// the MMA as an exact int32, the 6-bit scale multiplies it on the CUDA cores, the mins meet the activations'
// 32-element sums in four dp2a, and the float chain is the mat-vec kernels' — same bits.
//
// CTA = 64 weight rows (4 warps x 16) x NT*8 columns; K is walked two super-blocks at a time through a three-stage
// cp.async ring that holds the weight rows as they lie in memory (2 x 144 bytes per row and stage), the
// activation bytes, their 16-element sums and scales.  Row strides are padded by 16 bytes so that the 8 rows x 4
// lanes of a fragment load fall on 32 different banks.
// Fragments (PTX ISA, m16n8k32, lane = 4g + t):
//   A: a0 (row g, k 4t..4t+3)  a1 (row g+8, same k)  a2 (row g, k 16+4t..)  a3 (row g+8, k 16+4t..)
//   B: b0 (k 4t..4t+3, col g)  b1 (k 16+4t.., col g)
//   C: c0,c1 (row g, cols 2t, 2t+1)  c2,c3 (row g+8, same cols)
#include "common.cuh"
#include "kernels.h"

namespace emelb {

namespace {

constexpr int kWarpsM = 4, kTM = 16 * kWarpsM, kSbPerStage = 2, kStageK = kSbPerStage * QK_K, kStagesM = 3;
constexpr int kWRow = kSbPerStage * Q4_K_BYTES + 16;   // 304 bytes = 76 words: 76 g + t covers 32 banks
constexpr int kXRow = kStageK + 16;                    // 528 bytes = 132 words: 4 g + t
constexpr int kBsRow = kStageK / 16 * 2 + 16;          // 32 int16 sums of 16 elements, padded
constexpr int kThreadsM = 32 * kWarpsM;

template <int NT>
struct Q4Stage {
  uint8_t w[kTM][kWRow];
  int8_t x[NT * 8][kXRow];
  uint8_t bs[NT * 8][kBsRow];
  float dx[NT * 8][kSbPerStage];
};

__device__ __forceinline__ void mma_s8(int (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// the same instruction with a zero addend (no accumulator registers to clear)
__device__ __forceinline__ void mma_s8_z(int (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
               : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "r"(0));
}

// four 8 x 16-byte matrices from shared memory: lane l gives the address of row l % 8 of matrix l / 8; thread
// (g, t) receives bytes 4t .. 4t+3 of row g of each matrix -- the m16n8k32 operand fragments
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}

__device__ __forceinline__ int dp2a_lo_su(uint32_t pair, uint32_t bytes, int c) {
  int d;
  asm("dp2a.lo.s32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(pair), "r"(bytes), "r"(c));
  return d;
}
__device__ __forceinline__ int dp2a_hi_su(uint32_t pair, uint32_t bytes, int c) {
  int d;
  asm("dp2a.hi.s32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(pair), "r"(bytes), "r"(c));
  return d;
}

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void cp_async8(void* smem, const void* gmem) {
  const uint32_t s = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
  asm volatile("cp.async.ca.shared.global [%0], [%1], 8;\n" ::"r"(s), "l"(gmem) : "memory");
}

// the 6-bit scales and mins of a super-block as four words of four bytes: scales 0-3, 4-7, mins 0-3, 4-7
// (get_scale_min_k4, src/emel/kernel/detail.hpp:1066-1076)
struct ScaleWords { uint32_t sc_lo, sc_hi, mn_lo, mn_hi; };
__device__ __forceinline__ ScaleWords unpack_scales(const uint4& h) {
  ScaleWords s;
  s.sc_lo = h.y & 0x3f3f3f3fu;
  s.mn_lo = h.z & 0x3f3f3f3fu;
  s.sc_hi = (h.w & 0x0f0f0f0fu) | (((h.y >> 6) & 0x03030303u) << 4);
  s.mn_hi = ((h.w >> 4) & 0x0f0f0f0fu) | (((h.z >> 6) & 0x03030303u) << 4);
  return s;
}

template <int NT>
__global__ void __launch_bounds__(kThreadsM, 2) gemm_q4k_mma_kernel(const GemvArgs p, int ncols) {
  using Stage = Q4Stage<NT>;
  extern __shared__ __align__(16) unsigned char smem_q4m[];
  Stage* stages = reinterpret_cast<Stage*>(smem_q4m);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
  const int row0 = blockIdx.x * kTM;
  const int nstages = p.K / kStageK;

  // rows and columns past the edge are read from the last valid one (their results are never stored)
  auto issue = [&](int ks, Stage& st) {
    constexpr int kWPieces = kSbPerStage * Q4_K_BYTES / 16;   // 18
    for (int idx = tid; idx < kTM * kWPieces; idx += kThreadsM) {
      const int r = idx / kWPieces, piece = idx - r * kWPieces;
      const int row = min(row0 + r, p.M - 1);
      cp_async16(&st.w[r][16 * piece], p.W + (int64_t)row * p.row_bytes + (int64_t)ks * (kSbPerStage * Q4_K_BYTES) + 16 * piece);
    }
    constexpr int kXPieces = kStageK / 16;                    // 32
    for (int idx = tid; idx < NT * 8 * kXPieces; idx += kThreadsM) {
      const int c = idx / kXPieces, piece = idx - c * kXPieces;
      const int col = p.col0 + min(c, ncols - 1);
      cp_async16(&st.x[c][16 * piece], p.act.qs + (int64_t)col * p.act.col_stride_qs + (int64_t)ks * kStageK + 16 * piece);
    }
    constexpr int kBPieces = kStageK / 16 * 2 / 16;           // 4
    for (int idx = tid; idx < NT * 8 * kBPieces; idx += kThreadsM) {
      const int c = idx / kBPieces, piece = idx - c * kBPieces;
      const int col = p.col0 + min(c, ncols - 1);
      cp_async16(&st.bs[c][16 * piece], reinterpret_cast<const uint8_t*>(p.act.bsums + (int64_t)col * p.act.col_stride_bs + (int64_t)ks * (kStageK / 16)) + 16 * piece);
    }
    for (int c = tid; c < NT * 8; c += kThreadsM) {
      const int col = p.col0 + min(c, ncols - 1);
      cp_async8(&st.dx[c][0], p.act.d + (int64_t)col * p.act.col_stride_d + (int64_t)ks * kSbPerStage);
    }
    cp_async_commit();
  };

  float acc[NT][4];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt)
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[nt][i] = 0.0f;

#pragma unroll
  for (int s = 0; s < kStagesM - 1; ++s) {
    if (s < nstages) issue(s, stages[s]);
    else cp_async_commit();
  }
  const int ra = warp * 16 + g, rb = ra + 8;
  for (int ks = 0; ks < nstages; ++ks) {
    // the ring slot refilled here was read two turns ago; every warp has passed the barrier that ended that turn
    if (ks + kStagesM - 1 < nstages) issue(ks + kStagesM - 1, stages[(ks + kStagesM - 1) % kStagesM]);
    else cp_async_commit();
    cp_async_wait<kStagesM - 1>();
    __syncthreads();
    const Stage& st = stages[ks % kStagesM];
#pragma unroll
    for (int sb = 0; sb < kSbPerStage; ++sb) {
      const uint8_t* ba = &st.w[ra][sb * Q4_K_BYTES];
      const uint8_t* bb = &st.w[rb][sb * Q4_K_BYTES];
      const uint4 ha = *reinterpret_cast<const uint4*>(ba), hb = *reinterpret_cast<const uint4*>(bb);
      const ScaleWords sa = unpack_scales(ha), sw = unpack_scales(hb);
      int isum[NT][4];
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int i = 0; i < 4; ++i) isum[nt][i] = 0;
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        // bytes 32r .. 32r+31 of the quants: low nibbles = sub-block 2r, high nibbles = sub-block 2r+1
        const uint32_t wa0 = *reinterpret_cast<const uint32_t*>(ba + 16 + 32 * r + 4 * t);
        const uint32_t wa1 = *reinterpret_cast<const uint32_t*>(ba + 32 + 32 * r + 4 * t);
        const uint32_t wb0 = *reinterpret_cast<const uint32_t*>(bb + 16 + 32 * r + 4 * t);
        const uint32_t wb1 = *reinterpret_cast<const uint32_t*>(bb + 32 + 32 * r + 4 * t);
        const uint32_t scw_a = r < 2 ? sa.sc_lo : sa.sc_hi, scw_b = r < 2 ? sw.sc_lo : sw.sc_hi;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          const int j = 2 * r + half, sh = 16 * (r & 1) + 8 * half;
          const int sca = (int)((scw_a >> sh) & 0xffu), scb = (int)((scw_b >> sh) & 0xffu);
          const uint32_t af[4] = {(wa0 >> (4 * half)) & 0x0f0f0f0fu, (wb0 >> (4 * half)) & 0x0f0f0f0fu,
                                  (wa1 >> (4 * half)) & 0x0f0f0f0fu, (wb1 >> (4 * half)) & 0x0f0f0f0fu};
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) {
            const int8_t* xr = &st.x[nt * 8 + g][sb * QK_K + j * 32 + 4 * t];
            const uint32_t b0 = *reinterpret_cast<const uint32_t*>(xr), b1 = *reinterpret_cast<const uint32_t*>(xr + 16);
            int c[4] = {0, 0, 0, 0};
            mma_s8(c, af, b0, b1);
            isum[nt][0] += sca * c[0];
            isum[nt][1] += sca * c[1];
            isum[nt][2] += scb * c[2];
            isum[nt][3] += scb * c[3];
          }
        }
      }
      const float da = h2f((uint16_t)(ha.x & 0xffffu)), dmin_a = h2f((uint16_t)(ha.x >> 16));
      const float db = h2f((uint16_t)(hb.x & 0xffffu)), dmin_b = h2f((uint16_t)(hb.x >> 16));
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          const int col = nt * 8 + 2 * t + i;
          // the column's sixteen 16-element sums of this super-block -> eight 32-element sums, two per word
          const int4 s0 = *reinterpret_cast<const int4*>(&st.bs[col][sb * 32]);
          const int4 s1 = *reinterpret_cast<const int4*>(&st.bs[col][sb * 32 + 16]);
          const int w[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
          uint32_t pw[4];
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const int p0 = (int)(short)(w[2 * k] & 0xffff) + (w[2 * k] >> 16);
            const int p1 = (int)(short)(w[2 * k + 1] & 0xffff) + (w[2 * k + 1] >> 16);
            pw[k] = ((uint32_t)p0 & 0xffffu) | ((uint32_t)p1 << 16);
          }
          int ma = dp2a_lo_su(pw[0], sa.mn_lo, 0);
          ma = dp2a_hi_su(pw[1], sa.mn_lo, ma);
          ma = dp2a_lo_su(pw[2], sa.mn_hi, ma);
          ma = dp2a_hi_su(pw[3], sa.mn_hi, ma);
          int mb = dp2a_lo_su(pw[0], sw.mn_lo, 0);
          mb = dp2a_hi_su(pw[1], sw.mn_lo, mb);
          mb = dp2a_lo_su(pw[2], sw.mn_hi, mb);
          mb = dp2a_hi_su(pw[3], sw.mn_hi, mb);
          const float dx = st.dx[col][sb];
          const float va = __fmaf_rn(__fmul_rn(dx, da), (float)isum[nt][i], -__fmul_rn(__fmul_rn(dx, dmin_a), (float)ma));
          const float vb = __fmaf_rn(__fmul_rn(dx, db), (float)isum[nt][2 + i], -__fmul_rn(__fmul_rn(dx, dmin_b), (float)mb));
          acc[nt][i] = __fadd_rn(acc[nt][i], va);
          acc[nt][2 + i] = __fadd_rn(acc[nt][2 + i], vb);
        }
      }
    }
    __syncthreads();  // this slot is free for the copy issued at the top of the next turn but one
  }

  const int ya = row0 + ra, yb = row0 + rb;
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int c = nt * 8 + 2 * t + i;
      if (c >= ncols) continue;
      if (ya < p.M) p.y[(int64_t)ya * p.ldy + p.col0 + c] = acc[nt][i];
      if (yb < p.M) p.y[(int64_t)yb * p.ldy + p.col0 + c] = acc[nt][2 + i];
    }
  }
}

// ---- the 16-column kernel: 64 rows x 16 columns per tile, K split over the warps.
// A warp of the kernel above walks K alone, one super-block after the other, and is bound by its own instruction
// latency (about 0.7 us per super-block).  Here 16 warps = 4 row groups of 16 rows x 4 quarters of a stage of four
// super-blocks: warp (rg, kq) computes the 256 block values of rows rg*16.. x 16 columns for super-block kq of the
// stage and leaves them in shared memory; after a barrier thread i adds the four values of its two (row, column)
// elements to its running sums in ascending super-block order.  The float chain per element is therefore the
// one-warp kernel's (and the mat-vec kernels'), while four times as many warps stream a row.
// A CTA walks tiles blockIdx.x, + gridDim.x, ... with one copy ring that runs on across tile boundaries; it is
// launched with one CTA per tile, which measured faster than one CTA per SM.  Up to three matrices of one K (Q, K,
// V or gate, up) run in one launch: tiles are counted through the segments.
// The columns' 32-element activation sums (two 16-element sums each) are packed once per stage by the threads that
// copied them, two per word, as dp2a wants them.
// Two shapes of the kernel: RG = 4 row groups (64-row tiles, 16 warps, three stages, one CTA per SM) and RG = 2
// (32-row tiles, 8 warps, two stages, two CTAs per SM) for matrices whose 64-row tiles would not fill the GPU -- a
// CTA's walk along K is a chain of dependent turns, so more and smaller CTAs that interleave on an SM finish sooner.
constexpr int kSbPerStage16 = 4, kStageK16 = kSbPerStage16 * QK_K;
constexpr int kWPieces16 = kSbPerStage16 * Q4_K_BYTES / 16;                               // 36 per row
constexpr int kWSlots16 = 5;   // ceil(16 RG rows x 36 pieces / (128 RG threads)) = ceil(4.5): copies per thread, the last one half used
constexpr int kSmall16Factor = 8;   // fewer 64-row tiles than this many per SM: the 32-row shape
constexpr int kWRow16 = kSbPerStage16 * Q4_K_BYTES + 16;   // 592 bytes = 148 words: 20 g + t covers 32 banks
constexpr int kXRow16 = kStageK16 + 16;                    // 1040 bytes = 260 words: 4 g + t

template <int RG>
struct Q4Stage16 {
  uint8_t w[16 * RG][kWRow16];
  int8_t x[16][kXRow16];
  uint8_t bs[16][kSbPerStage16][32];     // raw 16-element sums: 16 int16 per column and super-block
  uint4 pw[16][kSbPerStage16 + 1];       // the same as eight 32-element sums, two per word (80-byte rows: 4 columns on 16 banks)
  float dx[16][kSbPerStage16];
};
template <int RG, int STAGES>
struct Q4Smem16 {
  Q4Stage16<RG> stage[STAGES];
  float table[2][RG][kSbPerStage16][256];   // [stage parity][row group][super-block of the stage][row * 16 + column]
};

struct Tile16 {
  const uint8_t* W;
  float* y;
  int M, row0;
};

template <int RG, int STAGES>
__global__ void __launch_bounds__(128 * RG, RG == 4 ? 1 : 2) gemm_q4k_mma16_kernel(const GemvArgs p, int ncols) {
  constexpr int kRows16 = 16 * RG, kThreads16 = 128 * RG, kStages16 = STAGES, kXPer = 1024 / kThreads16;
  using Q4Stage16 = Q4Stage16<RG>;
  extern __shared__ __align__(16) unsigned char smem_q4m16[];
  Q4Smem16<RG, STAGES>& sm = *reinterpret_cast<Q4Smem16<RG, STAGES>*>(smem_q4m16);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
  const int rg = warp >> 2, kq = warp & 3;
  const int nstages = p.K / kStageK16;
  const int nt0 = (p.M + kRows16 - 1) / kRows16, nt1 = (p.M2 + kRows16 - 1) / kRows16, nt2 = (p.M3 + kRows16 - 1) / kRows16;
  const int ntiles = nt0 + nt1 + nt2;
  const int my_tiles = ((int)blockIdx.x < ntiles) ? (ntiles - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
  const int total = my_tiles * nstages;   // stages this CTA walks

  auto tile_of = [&](int i) {
    int tile = blockIdx.x + i * gridDim.x;
    const int seg = tile < nt0 ? 0 : (tile < nt0 + nt1 ? 1 : 2);
    tile -= seg == 0 ? 0 : (seg == 1 ? nt0 : nt0 + nt1);
    Tile16 r;
    r.W = seg == 0 ? p.W : (seg == 1 ? p.W2 : p.W3);
    r.M = seg == 0 ? p.M : (seg == 1 ? p.M2 : p.M3);
    r.y = seg == 0 ? p.y : (seg == 1 ? p.y2 : p.y3);
    r.row0 = tile * kRows16;
    return r;
  };

  // this thread's copies of a stage (16-byte cp.async): tile-independent parts once, the weight rows per tile.
  // Bulk copies (cp.async.bulk, one per 576-byte row piece) were tried instead and ran at half the speed: 112 small
  // copies per stage and SM are more than the copy engine takes without stalling.
  // activation pieces tid, tid + threads, ...: 16 columns x 64 pieces of 16 bytes per stage
  const int8_t* xsrc[kXPer];
  int xdst[kXPer];
#pragma unroll
  for (int q = 0; q < kXPer; ++q) {
    const int idx = tid + q * kThreads16, xc = idx >> 6, xp = idx & 63;
    xsrc[q] = p.act.qs + (int64_t)(p.col0 + min(xc, ncols - 1)) * p.act.col_stride_qs + 16 * xp;
    xdst[q] = xc * kXRow16 + 16 * xp;
  }
  const int bcol = tid >> 2, bsb = tid & 3;                                   // tid < 64: 32 bytes of sums; 64 <= tid < 80: scales
  const uint8_t* bsrc = reinterpret_cast<const uint8_t*>(p.act.bsums + (int64_t)(p.col0 + min(bcol & 15, ncols - 1)) * p.act.col_stride_bs) + 32 * bsb;
  const float* dsrc = p.act.d + (int64_t)(p.col0 + min(tid & 15, ncols - 1)) * p.act.col_stride_d;
  int wdst[kWSlots16];
  int64_t wsrc[kWSlots16];
  Tile16 itile{};    // the tile the next issued stage belongs to
  int it_tile = -1;
  auto set_issue_tile = [&](int i) {
    itile = tile_of(i);
    it_tile = i;
#pragma unroll
    for (int sl = 0; sl < kWSlots16; ++sl) {
      const int idx = tid + sl * kThreads16;
      const int r = idx / kWPieces16, piece = idx - r * kWPieces16;
      wdst[sl] = r * kWRow16 + 16 * piece;
      wsrc[sl] = (int64_t)min(itile.row0 + r, itile.M - 1) * p.row_bytes + 16 * piece;
    }
  };
  auto issue = [&](int it) {   // stage it of this CTA's walk
    const int i = it / nstages, ks = it - i * nstages;
    if (i != it_tile) set_issue_tile(i);
    Q4Stage16& st = sm.stage[it % kStages16];
    const uint8_t* wbase = itile.W + (int64_t)ks * (kSbPerStage16 * Q4_K_BYTES);
#pragma unroll
    for (int sl = 0; sl < kWSlots16; ++sl)
      if (sl < kWSlots16 - 1 || tid < kRows16 * kWPieces16 - (kWSlots16 - 1) * kThreads16)
        cp_async16(&st.w[0][0] + wdst[sl], wbase + wsrc[sl]);
#pragma unroll
    for (int q = 0; q < kXPer; ++q) cp_async16(&st.x[0][0] + xdst[q], xsrc[q] + (int64_t)ks * kStageK16);
    if (tid < 64) {
      cp_async16(&st.bs[bcol][bsb][0], bsrc + (int64_t)ks * (kStageK16 / 8));
      cp_async16(&st.bs[bcol][bsb][16], bsrc + (int64_t)ks * (kStageK16 / 8) + 16);
    } else if (tid < 80) {
      cp_async16(&st.dx[tid & 15][0], dsrc + (int64_t)ks * kSbPerStage16);
    }
    cp_async_commit();
  };

  float acc[2] = {0.0f, 0.0f};   // elements tid and tid + threads of the tile's rows x 16 outputs
#pragma unroll
  for (int s = 0; s < kStages16 - 1; ++s) {
    if (s < total) issue(s);
    else cp_async_commit();
  }
  Tile16 ctile{};
  for (int it = 0; it < total; ++it) {
    const int i = it / nstages, ks = it - i * nstages;
    if (ks == 0) {
      ctile = tile_of(i);
      acc[0] = acc[1] = 0.0f;
    }
    cp_async_wait<kStages16 - 2>();   // this thread's copies of stage `it` have landed
    Q4Stage16& st = sm.stage[it % kStages16];
    if (tid < 64) {
      // 16-element sums -> eight 32-element sums, two per word (this thread copied these 32 bytes itself)
      const int4 s0 = *reinterpret_cast<const int4*>(&st.bs[bcol][bsb][0]);
      const int4 s1 = *reinterpret_cast<const int4*>(&st.bs[bcol][bsb][16]);
      const int w[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
      uint32_t pw[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int p0 = (int)(short)(w[2 * k] & 0xffff) + (w[2 * k] >> 16);
        const int p1 = (int)(short)(w[2 * k + 1] & 0xffff) + (w[2 * k + 1] >> 16);
        pw[k] = ((uint32_t)p0 & 0xffffu) | ((uint32_t)p1 << 16);
      }
      st.pw[bcol][bsb] = make_uint4(pw[0], pw[1], pw[2], pw[3]);
    }
    __syncthreads();   // stage `it` is complete for every thread; the slot refilled below was last read before this barrier
    if (it + kStages16 - 1 < total) issue(it + kStages16 - 1);
    else cp_async_commit();
    {
      const int sb = kq;
      const uint8_t* ba = &st.w[rg * 16 + g][sb * Q4_K_BYTES];
      const uint8_t* bb = ba + 8 * kWRow16;
      const uint4 ha = *reinterpret_cast<const uint4*>(ba), hb = *reinterpret_cast<const uint4*>(bb);
      const ScaleWords sa = unpack_scales(ha), sw = unpack_scales(hb);
      // operand fragments by ldmatrix: the weights' raw quant bytes (rows 0-7 / 8-15 x byte halves 0-15 / 16-31 of
      // a 32-byte span = sub-blocks 2r, 2r+1) and the activations of both column groups (bytes 0-15 / 16-31 of a
      // sub-block)
      const uint32_t wfrag = smem_addr(&st.w[rg * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)][sb * Q4_K_BYTES + 16 + 16 * (lane >> 4)]);
      const uint32_t xfrag = smem_addr(&st.x[(lane & 7) + 8 * (lane >> 4)][sb * QK_K + 16 * ((lane >> 3) & 1)]);
      int isum[2][4];
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int q = 0; q < 4; ++q) isum[nt][q] = 0;
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        uint32_t wq[4];
        ldsm_x4(wq, wfrag + 32 * r);
        const uint32_t scw_a = r < 2 ? sa.sc_lo : sa.sc_hi, scw_b = r < 2 ? sw.sc_lo : sw.sc_hi;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          const int j = 2 * r + half, sh = 16 * (r & 1) + 8 * half;
          const int sca = (int)((scw_a >> sh) & 0xffu), scb = (int)((scw_b >> sh) & 0xffu);
          const uint32_t af[4] = {(wq[0] >> (4 * half)) & 0x0f0f0f0fu, (wq[1] >> (4 * half)) & 0x0f0f0f0fu,
                                  (wq[2] >> (4 * half)) & 0x0f0f0f0fu, (wq[3] >> (4 * half)) & 0x0f0f0f0fu};
          uint32_t xb[4];   // {b0, b1} of columns 0-7, then of columns 8-15
          ldsm_x4(xb, xfrag + 32 * j);
#pragma unroll
          for (int nt = 0; nt < 2; ++nt) {
            int c[4];
            mma_s8_z(c, af, xb[2 * nt], xb[2 * nt + 1]);
            isum[nt][0] += sca * c[0];
            isum[nt][1] += sca * c[1];
            isum[nt][2] += scb * c[2];
            isum[nt][3] += scb * c[3];
          }
        }
      }
      const float da = h2f((uint16_t)(ha.x & 0xffffu)), dmin_a = h2f((uint16_t)(ha.x >> 16));
      const float db = h2f((uint16_t)(hb.x & 0xffffu)), dmin_b = h2f((uint16_t)(hb.x >> 16));
      float* tab = sm.table[it & 1][rg][kq];
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
        float va[2], vb[2];
#pragma unroll
        for (int q = 0; q < 2; ++q) {
          const int col = nt * 8 + 2 * t + q;
          const uint4 pw = st.pw[col][sb];
          int ma = dp2a_lo_su(pw.x, sa.mn_lo, 0);
          ma = dp2a_hi_su(pw.y, sa.mn_lo, ma);
          ma = dp2a_lo_su(pw.z, sa.mn_hi, ma);
          ma = dp2a_hi_su(pw.w, sa.mn_hi, ma);
          int mb = dp2a_lo_su(pw.x, sw.mn_lo, 0);
          mb = dp2a_hi_su(pw.y, sw.mn_lo, mb);
          mb = dp2a_lo_su(pw.z, sw.mn_hi, mb);
          mb = dp2a_hi_su(pw.w, sw.mn_hi, mb);
          const float dx = st.dx[col][sb];
          va[q] = __fmaf_rn(__fmul_rn(dx, da), (float)isum[nt][q], -__fmul_rn(__fmul_rn(dx, dmin_a), (float)ma));
          vb[q] = __fmaf_rn(__fmul_rn(dx, db), (float)isum[nt][2 + q], -__fmul_rn(__fmul_rn(dx, dmin_b), (float)mb));
        }
        *reinterpret_cast<float2*>(&tab[g * 16 + nt * 8 + 2 * t]) = make_float2(va[0], va[1]);
        *reinterpret_cast<float2*>(&tab[(g + 8) * 16 + nt * 8 + 2 * t]) = make_float2(vb[0], vb[1]);
      }
    }
    __syncthreads();   // the stage's block values are complete
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const int o = tid + e * kThreads16;
      const float* tab = &sm.table[it & 1][o >> 8][0][o & 255];
#pragma unroll
      for (int q = 0; q < kSbPerStage16; ++q) acc[e] = __fadd_rn(acc[e], tab[q * 256]);
    }
    if (ks == nstages - 1) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int o = tid + e * kThreads16;
        const int row = ctile.row0 + (o >> 4), col = o & 15;
        if (row < ctile.M && col < ncols) {
          const int64_t o16 = (int64_t)row * p.ldy + p.col0 + col;
          ctile.y[o16] = p.residual ? __fadd_rn(p.residual[o16], acc[e]) : acc[e];   // the residual belongs to the first matrix
        }
      }
    }
  }
  cp_async_wait<0>();
}

template <int RG, int STAGES>
cudaError_t launch_16_rg(const GemvArgs& a, int ncols, cudaStream_t st) {
  constexpr int kRows16 = 16 * RG;
  const int smem = (int)sizeof(Q4Smem16<RG, STAGES>);
  static thread_local unsigned configured = 0;  // one bit per device (one context, one lane per host thread)
  int dev = 0;
  cudaGetDevice(&dev);
  if (!(configured & (1u << (dev & 31)))) {
    const cudaError_t e = cudaFuncSetAttribute(gemm_q4k_mma16_kernel<RG, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    configured |= 1u << (dev & 31);
  }
  const int tiles = (a.M + kRows16 - 1) / kRows16 + (a.M2 + kRows16 - 1) / kRows16 + (a.M3 + kRows16 - 1) / kRows16;
  // one CTA per tile measured faster than one CTA per SM walking its tiles (36.8 against 41.1 us for 448 tiles)
  gemm_q4k_mma16_kernel<RG, STAGES><<<tiles, 128 * RG, smem, st>>>(a, ncols);
  return cudaGetLastError();
}

cudaError_t launch_16(const GemvArgs& a, int ncols, int sm_count, cudaStream_t st) {
  const int tiles64 = (a.M + 63) / 64 + (a.M2 + 63) / 64 + (a.M3 + 63) / 64;
  return tiles64 < kSmall16Factor * sm_count ? launch_16_rg<2, 2>(a, ncols, st) : launch_16_rg<4, 3>(a, ncols, st);
}

template <int NT>
cudaError_t launch_nt(const GemvArgs& a, int ncols, cudaStream_t st) {
  const int smem = (int)(kStagesM * sizeof(Q4Stage<NT>));
  static thread_local unsigned configured = 0;  // one bit per device (one context, one lane per host thread)
  int dev = 0;
  cudaGetDevice(&dev);
  if (!(configured & (1u << (dev & 31)))) {
    const cudaError_t e = cudaFuncSetAttribute(gemm_q4k_mma_kernel<NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    configured |= 1u << (dev & 31);
  }
  gemm_q4k_mma_kernel<NT><<<(a.M + kTM - 1) / kTM, kThreadsM, smem, st>>>(a, ncols);
  return cudaGetLastError();
}

}  // namespace

bool gemm_q4k_mma_supported(int type, const GemvArgs& a, int ncols) {
  if (type != T_Q4_K || ncols < kGemmQ4kMmaMinCols || ncols >= kGemmTcMinCols) return false;
  if (a.K % kStageK != 0 || a.pro_x || a.rope_cos || !a.act.bsums) return false;
  const bool grouped = a.W2 || a.W3;
  if (a.residual && (grouped || ncols > 16 || a.K % kStageK16 != 0)) return false;        // the 16-column kernel adds it on store
  if (grouped && (ncols > 16 || a.K % kStageK16 != 0)) return false;   // several matrices: the 16-column kernel only
  for (const uint8_t* w : {a.W, a.W2, a.W3})
    if (reinterpret_cast<uintptr_t>(w) % 16 != 0) return false;
  return a.row_bytes % 16 == 0 && reinterpret_cast<uintptr_t>(a.act.qs) % 16 == 0 &&
         a.act.col_stride_qs % 16 == 0 && reinterpret_cast<uintptr_t>(a.act.bsums) % 16 == 0 && a.act.col_stride_bs % 8 == 0 &&
         reinterpret_cast<uintptr_t>(a.act.d) % 16 == 0 && a.act.col_stride_d % 4 == 0;
}

cudaError_t launch_gemm_q4k_mma(const GemvArgs& a, int ncols, int sm_count, cudaStream_t st) {
  if (ncols <= 16 && a.K % kStageK16 == 0) return launch_16(a, ncols, sm_count, st);
  return ncols <= 16 ? launch_nt<2>(a, ncols, st) : launch_nt<4>(a, ncols, st);
}

}  // namespace emelb
