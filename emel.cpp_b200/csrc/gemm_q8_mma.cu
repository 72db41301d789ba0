// Many columns of Q8_0 / Q4_0 weights x Q8_0 activations on the tensor cores.
//
// Both formats scale every 32 weights on their own (src/emel/kernel/detail.hpp:3131-3153, 3252-3269:
// sumf += (float)sumi * (d_w * d_x), block after block), so a tensor-core instruction can cover exactly one block:
// mma.sync.m16n8k32 (s8 x s8 -> s32) gives the 32-term integer sums of 16 rows x 8 columns, and the CUDA
// cores apply the two scales and add the blocks up in ascending order with the reference's roundings — the
// same bits as the mat-vec kernels.  The scaling, 4 float operations per product and block, bounds the
// kernel, not the MMAs; a tcgen05 tile would only move the same scaling work behind a TMEM load.
//
// One CTA = 128 weight rows x 64 activation columns, 8 warps of 16 rows each; K is walked in chunks of 8
// blocks staged in shared memory as plain int8 rows (Q4_0 nibbles are widened to value - 8 while staging).
// Fragments (PTX ISA, m16n8k32, lane = 4g + t):
//   A: a0 (row g, k 4t..4t+3)  a1 (row g+8, same k)  a2 (row g, k 16+4t..)  a3 (row g+8, k 16+4t..)
//   B: b0 (k 4t..4t+3, col g)  b1 (k 16+4t.., col g)
//   C: c0,c1 (row g, cols 2t, 2t+1)  c2,c3 (row g+8, same cols)
#include <cstdlib>

#include "common.cuh"
#include "kernels.h"

namespace emelb {

namespace {

constexpr int kTM = 128, kTN = 64, kChunkBlocks = 8, kChunk = kChunkBlocks * QK32;
constexpr int kRowStride = kChunk + 16;  // bytes: fragment loads of 8 rows x 4 lanes hit 32 distinct banks
constexpr int kThreadsQ8 = 256;

struct Q8Smem {
  int8_t a[kTM][kRowStride];
  int8_t b[kTN][kRowStride];
  float dw[kTM][kChunkBlocks];
  float dx[kTN][kChunkBlocks];
};

__device__ __forceinline__ void mma_s8(int (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t ld16u(const uint8_t* p) { return (uint32_t)p[0] | ((uint32_t)p[1] << 8); }

template <int T>
__global__ void __launch_bounds__(kThreadsQ8, 2) gemm_q8_mma_kernel(const GemvArgs p, int ncols) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  Q8Smem& sm = *reinterpret_cast<Q8Smem*>(smem_raw);
  constexpr int BB = T == T_Q8_0 ? Q8_0_BYTES : Q4_0_BYTES;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
  const int row0 = blockIdx.x * kTM, c0 = blockIdx.y * kTN;

  float acc[kTN / 8][4];
#pragma unroll
  for (int nt = 0; nt < kTN / 8; ++nt)
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[nt][i] = 0.0f;

  for (int kc = 0; kc < p.K / kChunk; ++kc) {
    __syncthreads();  // the previous chunk's readers are done
    // weights: one (row, block) per thread and pass
    for (int idx = tid; idx < kTM * kChunkBlocks; idx += kThreadsQ8) {
      const int r = idx / kChunkBlocks, b = idx % kChunkBlocks;
      uint32_t w[8] = {0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u};
      float d = 0.0f;
      if (row0 + r < p.M) {
        const uint8_t* src = p.W + (int64_t)(row0 + r) * p.row_bytes + (int64_t)(kc * kChunkBlocks + b) * BB;
        d = h2f((uint16_t)ld16u(src));
        if constexpr (T == T_Q8_0) {
          // 32 int8 values at a 2-byte aligned address
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const uint16_t* h = reinterpret_cast<const uint16_t*>(src + 2 + 4 * i);
            w[i] = (uint32_t)h[0] | ((uint32_t)h[1] << 16);
          }
        } else {
          // 16 bytes: low nibbles = values 0..15, high nibbles = values 16..31, each minus 8
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const uint16_t* h = reinterpret_cast<const uint16_t*>(src + 2 + 4 * i);
            const uint32_t q = (uint32_t)h[0] | ((uint32_t)h[1] << 16);
            const uint32_t lo = q & 0x0f0f0f0fu, hi = (q >> 4) & 0x0f0f0f0fu;
            // per byte: value - 8 in two's complement (values 0..15, no borrow across bytes after the bias trick)
            w[i] = ((lo | 0x80808080u) - 0x08080808u) ^ 0x80808080u;
            w[4 + i] = ((hi | 0x80808080u) - 0x08080808u) ^ 0x80808080u;
          }
        }
      }
      uint4* dst = reinterpret_cast<uint4*>(&sm.a[r][b * QK32]);
      dst[0] = make_uint4(w[0], w[1], w[2], w[3]);
      dst[1] = make_uint4(w[4], w[5], w[6], w[7]);
      sm.dw[r][b] = d;
    }
    // activations: 16 bytes per thread and pass
    for (int idx = tid; idx < kTN * (kChunk / 16); idx += kThreadsQ8) {
      const int c = idx / (kChunk / 16), piece = idx % (kChunk / 16);
      uint4 v = make_uint4(0u, 0u, 0u, 0u);
      if (c0 + c < ncols)
        v = *reinterpret_cast<const uint4*>(p.act.qs + (int64_t)(p.col0 + c0 + c) * p.act.col_stride_qs + (int64_t)kc * kChunk + 16 * piece);
      *reinterpret_cast<uint4*>(&sm.b[c][16 * piece]) = v;
    }
    for (int idx = tid; idx < kTN * kChunkBlocks; idx += kThreadsQ8) {
      const int c = idx / kChunkBlocks, b = idx % kChunkBlocks;
      sm.dx[c][b] = c0 + c < ncols ? p.act.d[(int64_t)(p.col0 + c0 + c) * p.act.col_stride_d + kc * kChunkBlocks + b] : 0.0f;
    }
    __syncthreads();

    const int ra = warp * 16 + g, rb = ra + 8;
#pragma unroll
    for (int b = 0; b < kChunkBlocks; ++b) {
      uint32_t af[4];
      af[0] = *reinterpret_cast<const uint32_t*>(&sm.a[ra][b * QK32 + 4 * t]);
      af[1] = *reinterpret_cast<const uint32_t*>(&sm.a[rb][b * QK32 + 4 * t]);
      af[2] = *reinterpret_cast<const uint32_t*>(&sm.a[ra][b * QK32 + 16 + 4 * t]);
      af[3] = *reinterpret_cast<const uint32_t*>(&sm.a[rb][b * QK32 + 16 + 4 * t]);
      const float dwa = sm.dw[ra][b], dwb = sm.dw[rb][b];
#pragma unroll
      for (int nt = 0; nt < kTN / 8; ++nt) {
        const uint32_t b0 = *reinterpret_cast<const uint32_t*>(&sm.b[nt * 8 + g][b * QK32 + 4 * t]);
        const uint32_t b1 = *reinterpret_cast<const uint32_t*>(&sm.b[nt * 8 + g][b * QK32 + 16 + 4 * t]);
        int c[4] = {0, 0, 0, 0};
        mma_s8(c, af, b0, b1);
        const float dx0 = sm.dx[nt * 8 + 2 * t][b], dx1 = sm.dx[nt * 8 + 2 * t + 1][b];
        acc[nt][0] = __fadd_rn(acc[nt][0], __fmul_rn((float)c[0], __fmul_rn(dwa, dx0)));
        acc[nt][1] = __fadd_rn(acc[nt][1], __fmul_rn((float)c[1], __fmul_rn(dwa, dx1)));
        acc[nt][2] = __fadd_rn(acc[nt][2], __fmul_rn((float)c[2], __fmul_rn(dwb, dx0)));
        acc[nt][3] = __fadd_rn(acc[nt][3], __fmul_rn((float)c[3], __fmul_rn(dwb, dx1)));
      }
    }
  }

  const int ra = row0 + warp * 16 + g, rb = ra + 8;
#pragma unroll
  for (int nt = 0; nt < kTN / 8; ++nt) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int c = c0 + nt * 8 + 2 * t + i;
      if (c >= ncols) continue;
      if (ra < p.M) p.y[(int64_t)ra * p.ldy + p.col0 + c] = acc[nt][i];
      if (rb < p.M) p.y[(int64_t)rb * p.ldy + p.col0 + c] = acc[nt][2 + i];
    }
  }
}

template <int T>
cudaError_t launch_t(const GemvArgs& a, int ncols, cudaStream_t st) {
  const int smem = (int)sizeof(Q8Smem);
  cudaError_t e = cudaFuncSetAttribute(gemm_q8_mma_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return e;
  gemm_q8_mma_kernel<T><<<dim3((a.M + kTM - 1) / kTM, (ncols + kTN - 1) / kTN), kThreadsQ8, smem, st>>>(a, ncols);
  return cudaGetLastError();
}

}  // namespace

bool gemm_q8_mma_supported(int type, const GemvArgs& a, int ncols) {
  if (type != T_Q8_0 && type != T_Q4_0) return false;
  if (ncols < kGemmTcMinCols || a.K % kChunk != 0 || a.residual || a.W2 || a.W3 || a.pro_x || a.rope_cos) return false;
  return reinterpret_cast<uintptr_t>(a.W) % 2 == 0 && a.row_bytes % 2 == 0 && reinterpret_cast<uintptr_t>(a.act.qs) % 16 == 0 &&
         a.act.col_stride_qs % 16 == 0 && getenv("EMELB_NO_Q8_MMA") == nullptr;
}

cudaError_t launch_gemm_q8_mma(int type, const GemvArgs& a, int ncols, cudaStream_t st) {
  return type == T_Q8_0 ? launch_t<T_Q8_0>(a, ncols, st) : launch_t<T_Q4_0>(a, ncols, st);
}

}  // namespace emelb
