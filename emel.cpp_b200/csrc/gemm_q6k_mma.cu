// Nine or more columns of Q6_K weights x Q8_K activations (prompt batches and batch steps of models whose down /
// value / output projections are Q6_K, as in the usual Q4_K_M mix) on the legacy tensor path.
//
// Per 256-weight super-block and (row, column) the reference's value is
//   (dx*d) * (float)isum,  isum = sum_g scale_g * (dot16_g(q, x) - 32*bsum16_g)
// (src/emel/kernel/x86_64/actions.hpp:1036-1077; block layout src/emel/kernel/detail.hpp:592-629), added to the
// row sum in ascending block order.  A scale covers 16 weights, so one mma.sync.m16n8k16 (s8 x s8 -> s32) is one
// scale group of 16 rows against 8 columns.  The operand holds q - 32 (-32..31), which makes the group's integer
// dot16(q - 32, x) = dot16(q, x) - 32*bsum16 directly: the same integer, no block sums needed.  The int8 scale
// multiplies the MMA's exact int32 result on the CUDA cores and the float chain is the mat-vec kernels': same bits.
//
// CTA = WARPS x 16 weight rows x NT x 8 columns, one super-block of K per turn.  Q6_K blocks are 210 bytes, so a
// block starts at any even offset: cp.async brings for every row the 224-byte, 16-byte
// aligned window that covers the block (rows are 16-byte multiples -- K is a multiple of 2048 -- so the window
// never leaves the row), and a cooperative pass expands ql / qh from there into one int8 value per weight, K-major,
// which the A fragments are read from with ldmatrix.  Scales and d are read from the raw window.
// Fragments (PTX ISA, m16n8k16 .s8, lane = 4g + t):
//   A: a0 (row g, k 4t..4t+3)  a1 (row g+8, same k)     B: b0 (k 4t..4t+3, col g)
//   C: c0,c1 (row g, cols 2t, 2t+1)  c2,c3 (row g+8, same cols)
#include "common.cuh"
#include "kernels.h"

namespace emelb {

namespace {

constexpr int kRawWin = 224, kRawRow = kRawWin + 16;   // 240 bytes per row and stage
constexpr int kERow6 = QK_K + 16;                      // 272 bytes = 68 words: 8 rows x 16 bytes fall on 32 banks

// the activation side of a turn: NT x 8 columns of one super-block and their scales (double buffered)
template <int NT>
struct Q6XStage {
  int8_t x[NT * 8][kERow6];
  float dx[NT * 8];
};

__device__ __forceinline__ void mma_s8_k16(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%7,%7,%7,%7};"
               : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
               : "r"(a0), "r"(a1), "r"(b0), "r"(0));
}

__device__ __forceinline__ void ldsm6_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}

__device__ __forceinline__ uint32_t smem6(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void cp_async4(void* smem, const void* gmem) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(smem6(smem)), "l"(gmem) : "memory");
}

// 4 bytes at a 2-byte aligned shared-memory address
__device__ __forceinline__ uint32_t lds32_even(const uint8_t* p) {
  const uint16_t* h = reinterpret_cast<const uint16_t*>(p);
  return (uint32_t)h[0] | ((uint32_t)h[1] << 16);
}

// per byte: value (0..63) - 32 as int8
__device__ __forceinline__ uint32_t minus_32(uint32_t v) { return ((v | 0x80808080u) - 0x20202020u) ^ 0x80808080u; }

// Shared memory: a ring of RS raw windows per row (a window is refilled as soon as it has been expanded, so the copies
// run under the MMA loops), the expanded block, RS + 1 activation stages.  64 columns: RS = 1, 67 KB, three CTAs per
// SM, the MMA loop is long enough to cover one copy; 32 columns: RS = 2; 16 columns: RS = 1 again -- 42 KB, five CTAs
// per SM, which covers the copy better than a deeper ring in fewer CTAs did (6.73 against 6.76 ms for a batch-16 step).
template <int NT, int WARPS, int RS>
__global__ void __launch_bounds__(32 * WARPS) gemm_q6k_mma_kernel(const GemvArgs p, int ncols) {
  using XStage = Q6XStage<NT>;
  constexpr int kRows = 16 * WARPS, kThreads = 32 * WARPS, kCols = NT * 8;
  extern __shared__ __align__(16) unsigned char smem_q6m[];
  uint8_t (*raws)[kRows][kRawRow] = reinterpret_cast<uint8_t (*)[kRows][kRawRow]>(smem_q6m);
  int8_t (*e)[kERow6] = reinterpret_cast<int8_t (*)[kERow6]>(smem_q6m + RS * kRows * kRawRow);
  XStage* xs = reinterpret_cast<XStage*>(smem_q6m + RS * kRows * kRawRow + kRows * kERow6);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
  const int row0 = blockIdx.x * kRows, c0 = blockIdx.y * kCols;
  const int nsb = p.K / QK_K;

  // rows and columns past the edge are read from the last valid one (their results are never stored)
  auto issue = [&](int sb) {
    const int64_t win = ((int64_t)sb * Q6_K_BYTES) & ~(int64_t)15;   // the same for every row: rows are 16-byte multiples
    constexpr int kWPieces = kRawWin / 16;                            // 14
    for (int idx = tid; idx < kRows * kWPieces; idx += kThreads) {
      const int r = idx / kWPieces, piece = idx - r * kWPieces;
      const int row = min(row0 + r, p.M - 1);
      cp_async16(&raws[sb % RS][r][16 * piece], p.W + (int64_t)row * p.row_bytes + win + 16 * piece);
    }
    XStage& st = xs[sb % (RS + 1)];
    constexpr int kXPieces = QK_K / 16;                               // 16
    for (int idx = tid; idx < kCols * kXPieces; idx += kThreads) {
      const int c = idx / kXPieces, piece = idx - c * kXPieces;
      const int col = p.col0 + min(c0 + c, ncols - 1);
      cp_async16(&st.x[c][16 * piece], p.act.qs + (int64_t)col * p.act.col_stride_qs + (int64_t)sb * QK_K + 16 * piece);
    }
    for (int c = tid; c < kCols; c += kThreads) {
      const int col = p.col0 + min(c0 + c, ncols - 1);
      cp_async4(&st.dx[c], p.act.d + (int64_t)col * p.act.col_stride_d + sb);
    }
    cp_async_commit();
  };

  float acc[NT][4];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt)
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[nt][i] = 0.0f;

#pragma unroll
  for (int s0 = 0; s0 < RS; ++s0) {
    if (s0 < nsb) issue(s0);
    else cp_async_commit();
  }
  const int ra = warp * 16 + g, rb = ra + 8;
  // ldmatrix row addresses: A -- matrices (rows 0-7, group j), (rows 8-15, j), (rows 0-7, j+1), (rows 8-15, j+1);
  // B -- matrix m = group 4jj + m of the n-tile's eight columns
  const uint32_t a_lane = smem6(&e[warp * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)][16 * (lane >> 4)]);
  for (int sb = 0; sb < nsb; ++sb) {
    cp_async_wait<RS - 1>();
    __syncthreads();
    const XStage& st = xs[sb % (RS + 1)];
    uint8_t (*raw)[kRawRow] = raws[sb % RS];
    const int off = (sb * Q6_K_BYTES) & 15;         // of the block inside its window (even)
    // expand: item = (row, half n of the block, word i of that half's 32 byte positions) -> four words of q - 32.
    // A warp's 32 items are word i of rows R, R+2, R+4, R+6 for one n: 32 different banks for every load and store
    // (row strides of 60 and 68 words)
    for (int grp = warp; grp < kRows / 2; grp += WARPS) {
      const int n = grp & 1, r = 8 * (grp >> 2) + ((grp >> 1) & 1) + 2 * (lane >> 3), i = lane & 7;
      const uint8_t* blk = &raw[r][off];
      const uint32_t qa = lds32_even(blk + 64 * n + 4 * i), qb = lds32_even(blk + 64 * n + 32 + 4 * i);
      const uint32_t qh = lds32_even(blk + 128 + 32 * n + 4 * i);
      uint32_t* out = reinterpret_cast<uint32_t*>(&e[r][128 * n + 4 * i]);
      out[0] = minus_32((qa & 0x0f0f0f0fu) | ((qh & 0x03030303u) << 4));
      out[8] = minus_32((qb & 0x0f0f0f0fu) | (((qh >> 2) & 0x03030303u) << 4));
      out[16] = minus_32(((qa >> 4) & 0x0f0f0f0fu) | (((qh >> 4) & 0x03030303u) << 4));
      out[24] = minus_32(((qb >> 4) & 0x0f0f0f0fu) | (((qh >> 6) & 0x03030303u) << 4));
    }
    // the sixteen int8 scales and d of the two rows this thread holds results for
    uint32_t sa[4], sw[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      sa[k] = lds32_even(&raw[ra][off + 192 + 4 * k]);
      sw[k] = lds32_even(&raw[rb][off + 192 + 4 * k]);
    }
    const float da = h2f(*reinterpret_cast<const uint16_t*>(&raw[ra][off + 208]));
    const float db = h2f(*reinterpret_cast<const uint16_t*>(&raw[rb][off + 208]));
    __syncthreads();
    // this raw window is free, and so is the activation stage of the turn before: the copies for RS turns ahead
    // run under the MMA loops
    if (sb + RS < nsb) issue(sb + RS);
    else cp_async_commit();
    int isum[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int i = 0; i < 4; ++i) isum[nt][i] = 0;
#pragma unroll
    for (int jj = 0; jj < 4; ++jj) {
      uint32_t af[2][4];   // groups 4jj, 4jj+1 and 4jj+2, 4jj+3
      ldsm6_x4(af[0], a_lane + 64 * jj);
      ldsm6_x4(af[1], a_lane + 64 * jj + 32);
      int sca[4], scb[4];
#pragma unroll
      for (int m = 0; m < 4; ++m) {
        sca[m] = (int)(int8_t)((sa[jj] >> (8 * m)) & 0xffu);
        scb[m] = (int)(int8_t)((sw[jj] >> (8 * m)) & 0xffu);
      }
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        uint32_t bf[4];
        ldsm6_x4(bf, smem6(&st.x[nt * 8 + (lane & 7)][64 * jj + 16 * (lane >> 3)]));
#pragma unroll
        for (int m = 0; m < 4; ++m) {
          int c[4];
          mma_s8_k16(c, af[m >> 1][2 * (m & 1)], af[m >> 1][2 * (m & 1) + 1], bf[m]);
          isum[nt][0] += sca[m] * c[0];
          isum[nt][1] += sca[m] * c[1];
          isum[nt][2] += scb[m] * c[2];
          isum[nt][3] += scb[m] * c[3];
        }
      }
    }
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const float dx = st.dx[nt * 8 + 2 * t + i];
        acc[nt][i] = __fadd_rn(acc[nt][i], __fmul_rn(__fmul_rn(dx, da), (float)isum[nt][i]));
        acc[nt][2 + i] = __fadd_rn(acc[nt][2 + i], __fmul_rn(__fmul_rn(dx, db), (float)isum[nt][2 + i]));
      }
    }
    // no barrier here: the one at the top of the next turn separates this turn's reads of the expanded block and of
    // this activation stage from their next writers (the expansion of turn sb+1, the copies issued in turn sb+1)
  }

  const int ya = row0 + ra, yb = row0 + rb;
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int c = c0 + nt * 8 + 2 * t + i;
      if (c >= ncols) continue;
      if (ya < p.M) p.y[(int64_t)ya * p.ldy + p.col0 + c] = acc[nt][i];
      if (yb < p.M) p.y[(int64_t)yb * p.ldy + p.col0 + c] = acc[nt][2 + i];
    }
  }
}

template <int NT, int WARPS, int RS>
cudaError_t launch_q6(const GemvArgs& a, int ncols, cudaStream_t st) {
  constexpr int kRows = 16 * WARPS;
  const int smem = (int)((RS + 1) * sizeof(Q6XStage<NT>) + (size_t)kRows * (RS * kRawRow + kERow6));
  cudaError_t e = cudaFuncSetAttribute(gemm_q6k_mma_kernel<NT, WARPS, RS>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return e;
  gemm_q6k_mma_kernel<NT, WARPS, RS><<<dim3((a.M + kRows - 1) / kRows, (ncols + NT * 8 - 1) / (NT * 8)), 32 * WARPS, smem, st>>>(a, ncols);
  return cudaGetLastError();
}

}  // namespace

bool gemm_q6k_mma_supported(int type, const GemvArgs& a, int ncols) {
  if (type != T_Q6_K || ncols < kGemmMmaMinCols) return false;
  if (a.K % 2048 != 0 || a.residual || a.W2 || a.W3 || a.pro_x || a.rope_cos || a.join_in || a.join_out) return false;
  return reinterpret_cast<uintptr_t>(a.W) % 16 == 0 && a.row_bytes % 16 == 0 && reinterpret_cast<uintptr_t>(a.act.qs) % 16 == 0 &&
         a.act.col_stride_qs % 16 == 0;
}

cudaError_t launch_gemm_q6k_mma(const GemvArgs& a, int ncols, int sm_count, cudaStream_t st) {
  (void)sm_count;
  // column tile by column count: 16, 32 or 64 columns per CTA, 64 rows (32-row tiles for small grids measured no
  // faster: a CTA's walk along K is what takes the time there, and K cannot be split -- the sums are ordered)
  if (ncols <= 16) return launch_q6<2, 4, 1>(a, ncols, st);
  if (ncols <= 32) return launch_q6<4, 4, 2>(a, ncols, st);
  return launch_q6<8, 4, 1>(a, ncols, st);
}

}  // namespace emelb
