// Causal attention for a batch of prompt tokens over the f16 KV cache.
//
// The one-token kernels (attention.cu) re-read the whole cache for every query; a
// prompt of B tokens asks the same keys B times over.  Here one CTA owns a tile of
// query tokens and all the query heads that share one KV head (64 query rows in
// all), walks the cache in tiles of 64 positions staged in shared memory, and keeps
// the running maximum, sum and output rows in registers (f32 online softmax, the
// numerics of the split-KV decode kernel: queries rounded to f16 as the reference
// does, src/emel/kernel/detail.hpp:5238-5260; weights and accumulators in f32).
// Row r of the CTA = (query head r / QT of the group, token r % QT of the tile);
// token j of the batch sits at position pos0 + j and sees positions 0 .. pos0 + j.
#include <cuda_fp16.h>

#include <cmath>

#include "kernels.h"

namespace emelb {

namespace {

constexpr int kRows = 64;     // query rows per CTA
constexpr int kKT = 64;       // cache positions per tile

// ---------------------------------------------------------------------------------------------------------
// Scores and weighted sums run on the tensor cores (mma.sync m16n8k16, f16 operands, f32 accumulators).
// Scores are exact products of f16 values.  The softmax weights stay f32-accurate: each weight p is fed as
// two f16 operands, hi = f16(p) and lo = f16(p - hi), in two MMAs against the f16 V tile, so the only
// rounding left is the f32 accumulation (the 2e-5 bar of the fast attention holds).
// One warp = 16 query rows; lane = 4g + t.  Fragments (PTX ISA, m16n8k16):
//   A: a0 (row g, k 2t..2t+1)  a1 (row g+8, same k)  a2 (row g, k 2t+8..)  a3 (row g+8, k 2t+8..)
//   B: b0 (k 2t..2t+1, n g)    b1 (k 2t+8.., n g)
//   C: c0,c1 (row g, n 2t..2t+1)   c2,c3 (row g+8, n 2t..2t+1)
// so two adjacent score tiles (8 positions each) are, packed to f16, the A fragment of the P.V product.
constexpr int kMmaThreads = 128;

template <int D>
struct PrefillMmaSmem {
  static constexpr int kRowStride = D + 8;     // halves; rows 16 bytes x 17 apart: 8 rows of a fragment load cover all banks
  // Two K / V stages.  The query tile is needed only until the warps have taken their fragments into registers;
  // its memory then serves as the second K stage (kRows == kKT), so the double buffering costs one tile, not two
  __half q_k1[kRows][kRowStride];              // query tile, later K stage 1
  __half k0[kKT][kRowStride];
  __half v[2][kKT][kRowStride];                // row-major like K; ldmatrix.trans hands out the V fragments
};
static_assert(kRows == kKT, "the query tile doubles as a K stage");

// 16 bytes global -> shared without passing through registers; src_bytes = 0 fills the 16 bytes with zeros
__device__ __forceinline__ void cp_async16_zfill(void* smem, const void* gmem, int src_bytes) {
  const uint32_t s = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(src_bytes) : "memory");
}

// four 8x8 b16 matrices; lane l supplies the address of row l % 8 of matrix l / 8
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* row) {
  const uint32_t addr = static_cast<uint32_t>(__cvta_generic_to_shared(row));
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* row) {
  const uint32_t addr = static_cast<uint32_t>(__cvta_generic_to_shared(row));
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}

__device__ __forceinline__ void mma_f16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
  const __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&h);
}

template <int D>
__global__ void __launch_bounds__(kMmaThreads, 3) prefill_attention_mma_kernel(const PrefillAttnArgs a) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  PrefillMmaSmem<D>& sm = *reinterpret_cast<PrefillMmaSmem<D>*>(smem_raw);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
  const int n_rep = a.heads / a.kv_heads, QT = kRows / n_rep;
  // token tiles in descending order: a later tile walks more of the cache, and the long walks should start first
  const int kh = blockIdx.y, j0 = ((int)gridDim.x - 1 - (int)blockIdx.x) * QT, B = a.B;

  for (int idx = tid; idx < kRows * D; idx += kMmaThreads) {
    const int jt = idx % QT, d = (idx / QT) % D, rep = idx / (QT * D);
    const int j = j0 + jt;
    float val = 0.0f;
    if (j < B) val = a.q[((int64_t)(kh * n_rep + rep) * D + d) * B + j];
    sm.q_k1[rep * QT + jt][d] = __float2half_rn(val);
  }
  __syncthreads();

  // this warp's query fragments, kept in registers for the whole walk
  const int r0 = warp * 16 + g, r1 = r0 + 8;
  uint32_t qf[D / 16][4];
#pragma unroll
  for (int kk = 0; kk < D / 16; ++kk) {
    qf[kk][0] = *reinterpret_cast<const uint32_t*>(&sm.q_k1[r0][kk * 16 + 2 * t]);
    qf[kk][1] = *reinterpret_cast<const uint32_t*>(&sm.q_k1[r1][kk * 16 + 2 * t]);
    qf[kk][2] = *reinterpret_cast<const uint32_t*>(&sm.q_k1[r0][kk * 16 + 2 * t + 8]);
    qf[kk][3] = *reinterpret_cast<const uint32_t*>(&sm.q_k1[r1][kk * 16 + 2 * t + 8]);
  }
  int t_row[2];
  {
    const int ja = j0 + r0 % QT, jb = j0 + r1 % QT;
    t_row[0] = ja < B ? a.pos0 + ja + 1 : 0;
    t_row[1] = jb < B ? a.pos0 + jb + 1 : 0;
  }
  const int j_last = min(B, j0 + QT) - 1;
  const int t_cta = a.pos0 + j_last + 1;
  const int t_written = a.pos0 + B;

  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.0f, 0.0f};
  float o[D / 8][4];
#pragma unroll
  for (int dn = 0; dn < D / 8; ++dn)
#pragma unroll
    for (int i = 0; i < 4; ++i) o[dn][i] = 0.0f;
  const __half* kbase = a.k + (int64_t)kh * a.cache_head_stride;
  const __half* vbase = a.v + (int64_t)kh * a.cache_head_stride;

  // cache tile t0 .. t0+63 -> stage `buf`, asynchronously; rows the batch has not written yet are zero-filled
  auto issue = [&](int t0, int buf) {
    __half (*kdst)[PrefillMmaSmem<D>::kRowStride] = buf ? sm.q_k1 : sm.k0;
    for (int idx = tid; idx < kKT * (D / 8); idx += kMmaThreads) {
      const int tt = idx / (D / 8), c = idx % (D / 8);
      const bool live = t0 + tt < t_written;
      const int64_t off = (int64_t)(live ? t0 + tt : 0) * D + 8 * c;
      cp_async16_zfill(&kdst[tt][8 * c], kbase + off, live ? 16 : 0);
      cp_async16_zfill(&sm.v[buf][tt][8 * c], vbase + off, live ? 16 : 0);
    }
    asm volatile("cp.async.commit_group;\n" ::: "memory");
  };
  __syncthreads();   // every warp holds its query fragments: the query tile's memory may become K stage 1
  if (t_cta > 0) issue(0, 0);
  int buf = 0;
  for (int t0 = 0; t0 < t_cta; t0 += kKT, buf ^= 1) {
    // the other stage was read in the turn before; every warp has passed the barrier that ended that turn
    if (t0 + kKT < t_cta) {
      issue(t0 + kKT, buf ^ 1);
      asm volatile("cp.async.wait_group 1;\n" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;\n" ::: "memory");
    }
    __syncthreads();
    const __half (*ktile)[PrefillMmaSmem<D>::kRowStride] = buf ? sm.q_k1 : sm.k0;
    const __half (*vtile)[PrefillMmaSmem<D>::kRowStride] = sm.v[buf];

    // scores of 16 rows x 64 positions
    float s[kKT / 8][4];
#pragma unroll
    for (int nt = 0; nt < kKT / 8; ++nt) {
#pragma unroll
      for (int i = 0; i < 4; ++i) s[nt][i] = 0.0f;
      // K fragments of two 16-dim steps per load: matrices (dims kk*16..+7, +8..+15, (kk+1)*16..+7, +8..+15)
#pragma unroll
      for (int kk = 0; kk < D / 16; kk += 2) {
        uint32_t kb[4];
        ldmatrix_x4(kb, &ktile[nt * 8 + (lane & 7)][kk * 16 + ((lane >> 3) & 1) * 8 + (lane >> 4) * 16]);
        mma_f16(s[nt], qf[kk], kb[0], kb[1]);
        mma_f16(s[nt], qf[kk + 1], kb[2], kb[3]);
      }
    }

    // online softmax: thread holds rows r0 (values 0,1) and r1 (values 2,3); 4 lanes share a row
    float keep[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      float mx = -INFINITY;
#pragma unroll
      for (int nt = 0; nt < kKT / 8; ++nt)
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          const bool live = t0 + nt * 8 + 2 * t + i < t_row[h];
          float& v = s[nt][2 * h + i];
          v = live ? v * a.scale : -INFINITY;
          mx = fmaxf(mx, v);
        }
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      const float m_new = fmaxf(m[h], mx);
      keep[h] = m_new == -INFINITY ? 1.0f : expf(m[h] - m_new);
      float sum = 0.0f;
#pragma unroll
      for (int nt = 0; nt < kKT / 8; ++nt)
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          float& v = s[nt][2 * h + i];
          v = v == -INFINITY ? 0.0f : expf(v - m_new);
          sum += v;
        }
      sum += __shfl_xor_sync(0xffffffffu, sum, 1);
      sum += __shfl_xor_sync(0xffffffffu, sum, 2);
      l[h] = l[h] * keep[h] + sum;
      m[h] = m_new;
    }
#pragma unroll
    for (int dn = 0; dn < D / 8; ++dn) {
      o[dn][0] *= keep[0];
      o[dn][1] *= keep[0];
      o[dn][2] *= keep[1];
      o[dn][3] *= keep[1];
    }

    // O += P V, 16 positions per step, weights as hi + lo
#pragma unroll
    for (int jj = 0; jj < kKT / 16; ++jj) {
      uint32_t hi[4], lo[4];
#pragma unroll
      for (int part = 0; part < 2; ++part) {        // score tiles 2jj and 2jj + 1
        const float* p = s[2 * jj + part];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const __half2 ph = __floats2half2_rn(p[2 * h], p[2 * h + 1]);
          const float2 back = __half22float2(ph);
          hi[2 * part + h] = *reinterpret_cast<const uint32_t*>(&ph);
          lo[2 * part + h] = pack_half2(p[2 * h] - back.x, p[2 * h + 1] - back.y);
        }
      }
      // V fragments of two 8-dim column tiles per load, transposed on the way out of shared memory:
      // matrices (positions jj*16..+7 | +8..+15) x (dims dn*8..+7 | (dn+1)*8..+7)
#pragma unroll
      for (int dn = 0; dn < D / 8; dn += 2) {
        uint32_t vb[4];
        ldmatrix_x4_trans(vb, &vtile[jj * 16 + (lane & 7) + ((lane >> 3) & 1) * 8][(dn + (lane >> 4)) * 8]);
        mma_f16(o[dn], hi, vb[0], vb[1]);
        mma_f16(o[dn], lo, vb[0], vb[1]);
        mma_f16(o[dn + 1], hi, vb[2], vb[3]);
        mma_f16(o[dn + 1], lo, vb[2], vb[3]);
      }
    }
    __syncthreads();   // this stage is free for the copy issued at the top of the next turn
  }

#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int row = h == 0 ? r0 : r1, rep = row / QT, j = j0 + row % QT;
    if (j >= B) continue;
    const float inv = l[h] > 0.0f ? 1.0f / l[h] : 0.0f;
    float* out = a.dst + ((int64_t)(kh * n_rep + rep) * D) * B + j;
#pragma unroll
    for (int dn = 0; dn < D / 8; ++dn) {
      out[(int64_t)(dn * 8 + 2 * t) * B] = o[dn][2 * h] * inv;
      out[(int64_t)(dn * 8 + 2 * t + 1) * B] = o[dn][2 * h + 1] * inv;
    }
  }
}

template <int D>
cudaError_t launch_d(const PrefillAttnArgs& a, cudaStream_t st) {
  const int n_rep = a.heads / a.kv_heads, QT = kRows / n_rep;
  const dim3 grid((a.B + QT - 1) / QT, a.kv_heads);
  const int smem = (int)sizeof(PrefillMmaSmem<D>);
  cudaError_t e = cudaFuncSetAttribute(prefill_attention_mma_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return e;
  prefill_attention_mma_kernel<D><<<grid, kMmaThreads, smem, st>>>(a);
  return cudaGetLastError();
}

}  // namespace

bool prefill_attention_supported(const PrefillAttnArgs& a) {
  if (a.head_dim != 64 && a.head_dim != 128) return false;
  if (a.kv_heads <= 0 || a.heads % a.kv_heads != 0) return false;
  const int n_rep = a.heads / a.kv_heads;
  if (n_rep > kRows || kRows % n_rep != 0) return false;
  return reinterpret_cast<uintptr_t>(a.k) % 16 == 0 && reinterpret_cast<uintptr_t>(a.v) % 16 == 0 &&
         (a.cache_head_stride * 2) % 16 == 0;
}

cudaError_t launch_prefill_attention(const PrefillAttnArgs& a, cudaStream_t st) {
  return a.head_dim == 64 ? launch_d<64>(a, st) : launch_d<128>(a, st);
}

}  // namespace emelb
