// Decode GEMV / small-batch GEMM over GGUF block-quantized weight rows:
//   y[i*ldy + j] = sum_k W[i][k] * x_j[k]        (W: Q4_K | Q6_K | Q8_0 | Q4_0,
//                                                 x_j: Q8_K / Q8_0 planes)
// Replaces the row-dot loops of the reference's op_mul_mat
// (src/emel/kernel/detail.hpp:2846-2942, 3062-3153, 3252-3269, 3356-3571;
//  src/emel/kernel/x86_64/actions.hpp:763-1107, 1186-1326).
//
// This file holds the dispatch (launch_gemv), the generic kernel for shapes the
// streaming kernels do not take (K not a multiple of 2048, unaligned rows) and the
// argmax helpers; the streaming kernels are in gemv2.cu, the many-column
// tensor-core kernels in gemm_tc.cu and gemm_q8_mma.cu.
//
// Float order, all kernels.  The integers of a block are exact whatever the order;
// the f32 part follows the reference's x86 route literally: one value per block —
// fma(d*dx, isum, -(dmin*dx)*msum) for Q4_K, (d*dx)*isum for Q6_K, sumi*(dw*dx) for
// Q8_0/Q4_0 — added to the row sum block after block in ascending order
// (dot_*_row_avx2_fma, src/emel/kernel/x86_64/actions.hpp:876-896, 899-927,
// 999-1027, 1087-1107).  The result equals the reference's AVX2 output bit for bit
// (and its scalar output for Q8_0/Q4_0, whose two routes agree).
#include <cstdlib>

#include "common.cuh"
#include "kernels.h"

namespace emelb {

namespace {

constexpr int CHUNK = 2048;  // weights per row per pipeline item

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
  return launch_gemv_stream2(T, a, ncols, argmax, sm_count, st, launches, grid_out);
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
  return a.tc_ws && gemm_tc_supported(type, a.K, ncols, a.W, a.row_bytes, a.act) &&
         gemm_tc_workspace_bytes(a.K, ncols) <= a.tc_ws_bytes;
}

cudaError_t launch_gemv(int type, const GemvArgs& a, int ncols, bool argmax, int sm_count, cudaStream_t st,
                        int* launches) {
  // many columns of Q8_0 / Q4_0: one tensor-core instruction per 32-weight block (gemm_q8_mma.cu)
  if (!argmax && gemm_q8_mma_supported(type, a, ncols)) {
    ++*launches;
    return launch_gemm_q8_mma(type, a, ncols, sm_count, st);
  }
  // a handful of columns of Q4_K (several sequences decoding together): mma.sync per sub-block (gemm_q4k_mma.cu)
  if (!argmax && gemm_q4k_mma_supported(type, a, ncols)) {
    ++*launches;
    return launch_gemm_q4k_mma(a, ncols, sm_count, st);
  }
  // nine or more columns of Q6_K: mma.sync per 16-weight scale group (gemm_q6k_mma.cu)
  if (!argmax && gemm_q6k_mma_supported(type, a, ncols)) {
    ++*launches;
    return launch_gemm_q6k_mma(a, ncols, sm_count, st);
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
