// Many columns of Q8_0 / Q4_0 weights x Q8_0 activations on the tensor cores.
//
// Both formats scale every 32 weights on their own (src/emel/kernel/detail.hpp:3131-3153, 3252-3269:
// sumf += (float)sumi * (d_w * d_x), block after block), so a tensor-core instruction can cover exactly one block:
// mma.sync.m16n8k32 (s8 x s8 -> s32) gives the 32-term integer sums of 16 rows x 8 columns, and the CUDA
// cores apply the two scales and add the blocks up in ascending order with the reference's roundings — the
// same bits as the mat-vec kernels — two columns per instruction on the packed f32x2 pipe.  The scaling, 4 float operations per product and block, bounds the
// kernel, not the MMAs; a tcgen05 tile would only move the same scaling work behind a TMEM load.
//
// One CTA = 128 (or, for small grids, 64) weight rows x 64 activation columns, one warp per 16 rows; K is walked in chunks of 8
// blocks through a two-stage cp.async ring.  Weight rows are staged as they lie in memory (scale + quants,
// 34 or 18 bytes per block) and the A fragments are read from there with 2-byte loads (Q4_0 nibbles are
// widened to value - 8 in registers), so staging is pure asynchronous copying.
// Fragments (PTX ISA, m16n8k32, lane = 4g + t):
//   A: a0 (row g, k 4t..4t+3)  a1 (row g+8, same k)  a2 (row g, k 16+4t..)  a3 (row g+8, k 16+4t..)
//   B: b0 (k 4t..4t+3, col g)  b1 (k 16+4t.., col g)
//   C: c0,c1 (row g, cols 2t, 2t+1)  c2,c3 (row g+8, same cols)
#include <cstdlib>

#include "common.cuh"
#include "kernels.h"

namespace emelb {

namespace {

constexpr int kChunkBlocks = 8, kChunk = kChunkBlocks * QK32;
constexpr int kRowStride = kChunk + 16;  // bytes: fragment loads of 8 rows x 4 lanes hit 32 distinct banks

// One stage of the ring: the weight rows as they lie in memory (8 blocks = 272 B of Q8_0 or 144 B of Q4_0 per
// row, copied 16 bytes at a time by cp.async; both row strides put 8 rows x 4 lanes on distinct banks), the
// activation rows and their block scales.
template <int T, int WARPS, int NT>
struct Q8Stage {
  static constexpr int kTN = NT * 8;
  static constexpr int kTM = 16 * WARPS;
  static constexpr int kBB = T == T_Q8_0 ? Q8_0_BYTES : Q4_0_BYTES;
  static constexpr int kRaw = kChunkBlocks * kBB;
  uint8_t a[kTM][kRaw];
  int8_t b[kTN][kRowStride];
  float dx[kChunkBlocks][kTN];   // block-major: the scales of two neighbouring columns are one 8-byte load
};

__device__ __forceinline__ void mma_s8(int (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void cp_async4_q8(void* smem, const void* gmem) {
  const uint32_t s = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(s), "l"(gmem) : "memory");
}

// Two IEEE round-to-nearest f32 operations per instruction (sm_100 packed arithmetic), lane for lane the scalar
// result.  One trap, measured: a mul.rn.f32x2 whose only use is an add.rn.f32x2 comes out of ptxas (12.9) as one
// fused multiply-add -- a single rounding -- in spite of the .rn modifiers and of -fmad=false.  The sum is therefore
// written as fma(prod, 1.0, acc) with a 1.0 the assembler cannot see through: prod * 1 + acc rounds once, exactly as
// prod + acc does, and the product keeps its own rounding
__device__ __forceinline__ unsigned long long pack_f32x2(float lo, float hi) {
  unsigned long long r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ unsigned long long mul_f32x2(unsigned long long a, unsigned long long b) {
  unsigned long long r;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ unsigned long long fma_f32x2(unsigned long long a, unsigned long long b, unsigned long long c) {
  unsigned long long r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}
__device__ __forceinline__ float2 unpack_f32x2(unsigned long long v) {
  float2 r;
  asm("mov.b64 {%0, %1}, %2;" : "=f"(r.x), "=f"(r.y) : "l"(v));
  return r;
}

// 4 bytes at a 2-byte aligned shared-memory address
__device__ __forceinline__ uint32_t lds32_h(const uint8_t* p) {
  const uint16_t* h = reinterpret_cast<const uint16_t*>(p);
  return (uint32_t)h[0] | ((uint32_t)h[1] << 16);
}
// per byte: nibble value (0..15) - 8 as int8
__device__ __forceinline__ uint32_t nibbles_minus_8(uint32_t v) { return ((v | 0x80808080u) - 0x08080808u) ^ 0x80808080u; }

// NT x 8 columns per CTA (8 .. 64: few columns are a memory-bound walk over the weights, so narrow tiles with a deeper
// ring and more CTAs per SM), STAGES ring slots; one warp per 16 rows
template <int T, int WARPS, int NT, int STAGES>
__global__ void __launch_bounds__(32 * WARPS) gemm_q8_mma_kernel(const GemvArgs p, int ncols) {
  using Stage = Q8Stage<T, WARPS, NT>;
  constexpr int kTM = Stage::kTM, kThreadsQ8 = 32 * WARPS, kTN = NT * 8, NTW = NT, cgrp = 0;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  Stage* stages = reinterpret_cast<Stage*>(smem_raw);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
  const int row0 = blockIdx.x * kTM, c0 = blockIdx.y * kTN;
  const int chunks = p.K / kChunk;

  // rows and columns past the edge are read from the last valid one (their results are never stored)
  auto issue = [&](int kc, Stage& st) {
    constexpr int kPieces = Stage::kRaw / 16;
    for (int idx = tid; idx < kTM * kPieces; idx += kThreadsQ8) {
      const int r = idx / kPieces, piece = idx % kPieces;
      const int row = min(row0 + r, p.M - 1);
      cp_async16(&st.a[r][16 * piece], p.W + (int64_t)row * p.row_bytes + (int64_t)kc * Stage::kRaw + 16 * piece);
    }
    for (int idx = tid; idx < kTN * (kChunk / 16); idx += kThreadsQ8) {
      const int c = idx / (kChunk / 16), piece = idx % (kChunk / 16);
      const int col = p.col0 + min(c0 + c, ncols - 1);
      cp_async16(&st.b[c][16 * piece], p.act.qs + (int64_t)col * p.act.col_stride_qs + (int64_t)kc * kChunk + 16 * piece);
    }
    for (int idx = tid; idx < kTN * kChunkBlocks; idx += kThreadsQ8) {
      const int c = idx / kChunkBlocks, b = idx - c * kChunkBlocks;
      const int col = p.col0 + min(c0 + c, ncols - 1);
      cp_async4_q8(&st.dx[b][c], p.act.d + (int64_t)col * p.act.col_stride_d + kc * kChunkBlocks + b);
    }
    cp_async_commit();
  };

  // results as pairs of neighbouring columns: [0] row g, [1] row g+8.  The scaling runs on the packed f32x2
  // instructions (two IEEE-rounded operations per instruction: the same bits as the scalar chain)
  unsigned long long acc[NTW][2];
#pragma unroll
  for (int nt = 0; nt < NTW; ++nt) acc[nt][0] = acc[nt][1] = 0ull;

#pragma unroll
  for (int s0 = 0; s0 < STAGES - 1; ++s0) {
    if (s0 < chunks) issue(s0, stages[s0]);
    else cp_async_commit();
  }
  const int ra = warp * 16 + g, rb = ra + 8;
  // 1.0 in both lanes, as a value the assembler cannot know: prod * 1 + acc rounds once, exactly as prod + acc does
  const float one = p.K > 0 ? 1.0f : 2.0f;
  const unsigned long long one2 = pack_f32x2(one, one);
  for (int kc = 0; kc < chunks; ++kc) {
    // the slot refilled here was read in the turn before; every warp has passed the barrier that ended it
    if (kc + STAGES - 1 < chunks) issue(kc + STAGES - 1, stages[(kc + STAGES - 1) % STAGES]);
    else cp_async_commit();
    cp_async_wait<STAGES - 1>();
    __syncthreads();
    const Stage& st = stages[kc % STAGES];
#pragma unroll
    for (int b = 0; b < kChunkBlocks; ++b) {
      const uint8_t* ba = &st.a[ra][b * Stage::kBB];
      const uint8_t* bb = &st.a[rb][b * Stage::kBB];
      const float dwa = h2f(*reinterpret_cast<const uint16_t*>(ba)), dwb = h2f(*reinterpret_cast<const uint16_t*>(bb));
      const unsigned long long dwa2 = pack_f32x2(dwa, dwa), dwb2 = pack_f32x2(dwb, dwb);
      uint32_t af[4];
      if constexpr (T == T_Q8_0) {
        af[0] = lds32_h(ba + 2 + 4 * t);
        af[1] = lds32_h(bb + 2 + 4 * t);
        af[2] = lds32_h(ba + 2 + 16 + 4 * t);
        af[3] = lds32_h(bb + 2 + 16 + 4 * t);
      } else {
        // bytes 4t..4t+3 of the block: low nibbles = values 4t.., high nibbles = values 16+4t..
        const uint32_t qa = lds32_h(ba + 2 + 4 * t), qb = lds32_h(bb + 2 + 4 * t);
        af[0] = nibbles_minus_8(qa & 0x0f0f0f0fu);
        af[1] = nibbles_minus_8(qb & 0x0f0f0f0fu);
        af[2] = nibbles_minus_8((qa >> 4) & 0x0f0f0f0fu);
        af[3] = nibbles_minus_8((qb >> 4) & 0x0f0f0f0fu);
      }
#pragma unroll
      for (int nt = 0; nt < NTW; ++nt) {
        const int cb = (cgrp * NTW + nt) * 8;   // first column of this n-tile inside the CTA's tile
        const uint32_t b0 = *reinterpret_cast<const uint32_t*>(&st.b[cb + g][b * QK32 + 4 * t]);
        const uint32_t b1 = *reinterpret_cast<const uint32_t*>(&st.b[cb + g][b * QK32 + 16 + 4 * t]);
        int c[4] = {0, 0, 0, 0};
        mma_s8(c, af, b0, b1);
        const unsigned long long dx = *reinterpret_cast<const unsigned long long*>(&st.dx[b][cb + 2 * t]);
        acc[nt][0] = fma_f32x2(mul_f32x2(pack_f32x2((float)c[0], (float)c[1]), mul_f32x2(dwa2, dx)), one2, acc[nt][0]);
        acc[nt][1] = fma_f32x2(mul_f32x2(pack_f32x2((float)c[2], (float)c[3]), mul_f32x2(dwb2, dx)), one2, acc[nt][1]);
      }
    }
    __syncthreads();  // this stage is free for the copy issued at the top of the next turn
  }

  const int ya = row0 + ra, yb = row0 + rb;
#pragma unroll
  for (int nt = 0; nt < NTW; ++nt) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int c = c0 + (cgrp * NTW + nt) * 8 + 2 * t + i;
      if (c >= ncols) continue;
      const float2 va = unpack_f32x2(acc[nt][0]), vb = unpack_f32x2(acc[nt][1]);
      if (ya < p.M) p.y[(int64_t)ya * p.ldy + p.col0 + c] = i ? va.y : va.x;
      if (yb < p.M) p.y[(int64_t)yb * p.ldy + p.col0 + c] = i ? vb.y : vb.x;
    }
  }
}

template <int T, int WARPS, int NT, int STAGES>
cudaError_t launch_w(const GemvArgs& a, int ncols, cudaStream_t st) {
  constexpr int kTM = 16 * WARPS, kTN = NT * 8;
  const int smem = (int)(STAGES * sizeof(Q8Stage<T, WARPS, NT>));
  cudaError_t e = cudaFuncSetAttribute(gemm_q8_mma_kernel<T, WARPS, NT, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return e;
  gemm_q8_mma_kernel<T, WARPS, NT, STAGES><<<dim3((a.M + kTM - 1) / kTM, (ncols + kTN - 1) / kTN), 32 * WARPS, smem, st>>>(a, ncols);
  return cudaGetLastError();
}

// Many columns: 64-column tiles, 128 rows (64 while the 128-row grid would leave SMs without a CTA pair), two stages.
// Few columns: 8 / 16 / 32 / 64-column tiles of 64 rows with a deeper ring.  (Spreading a tile's columns over two or
// four warps per row group measured slower at 32 and 64 columns: 45.8 against 35.8 us and 62.0 against 56.2 us for
// 14336 x 4096 -- the kernel is bound by instructions per MMA, not by warps in flight)
template <int T>
cudaError_t launch_t(const GemvArgs& a, int ncols, int sm_count, cudaStream_t st) {
  if (ncols <= 8) return launch_w<T, 4, 1, 4>(a, ncols, st);
  if (ncols <= 16) return launch_w<T, 4, 2, 4>(a, ncols, st);
  if (ncols <= 32) return launch_w<T, 4, 4, 3>(a, ncols, st);
  const int64_t big = (int64_t)((a.M + 127) / 128) * ((ncols + 63) / 64);
  return big >= 2 * (int64_t)sm_count ? launch_w<T, 8, 8, 2>(a, ncols, st) : launch_w<T, 4, 8, 3>(a, ncols, st);
}

}  // namespace

bool gemm_q8_mma_supported(int type, const GemvArgs& a, int ncols) {
  if (type != T_Q8_0 && type != T_Q4_0) return false;
  if (ncols < kGemmQ8MmaMinCols || a.K % kChunk != 0 || a.residual || a.W2 || a.W3 || a.pro_x || a.rope_cos || a.join_in || a.join_out) return false;
  return reinterpret_cast<uintptr_t>(a.W) % 16 == 0 && a.row_bytes % 16 == 0 && reinterpret_cast<uintptr_t>(a.act.qs) % 16 == 0 &&
         a.act.col_stride_qs % 16 == 0 && reinterpret_cast<uintptr_t>(a.act.d) % 16 == 0;
}

cudaError_t launch_gemm_q8_mma(int type, const GemvArgs& a, int ncols, int sm_count, cudaStream_t st) {
  return type == T_Q8_0 ? launch_t<T_Q8_0>(a, ncols, sm_count, st) : launch_t<T_Q4_0>(a, ncols, sm_count, st);
}

}  // namespace emelb
