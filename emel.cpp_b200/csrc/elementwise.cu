// The element-wise steps between the matrix products of one decoder layer, as
// the reference's generator computes them (src/emel/text/generator/detail.hpp):
//   rms_norm                    :2735-2756   (f64 sum of f32 squares)
//   apply_rope_pairing          :2905-2936   (adjacent or half-split pairs)
//   store_attention_kv_cache    :3294-3332   (K, V rounded to f16)
//   silu(gate) * up             :2967-2973, 3911-3913 (expf with the host libm's bits)
//   copy_tensor_row             :819-872     (embedding row -> f32)
// Each kernel also emits what the next matrix product consumes (the quantized
// activation planes), so a layer is a short chain of launches.  Compiled with
// -fmad=false: every product and sum rounds as written in the reference.
#include "expf_exact.h"
#include "quant_device.cuh"
#include "peer_join.cuh"

namespace emelb {

namespace {

__device__ __forceinline__ double warp_sum_f64(double v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// ---- out = (x * 1/sqrt(mean(x^2) + eps)) * w ; optionally quantized for the
// consumer family (FAMILY 0: none, 1: Q8_K planes, 2: Q8_0 planes).  One CTA.
template <int FAMILY>
__global__ void __launch_bounds__(1024)
rms_norm_kernel(const float* __restrict__ x, const float* __restrict__ w, float eps, int n, float* out, ActPlanesMut planes) {
  pdl_trigger();
  pdl_wait();
  __shared__ double s_part[32];
  __shared__ float s_scale;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
  double acc = 0.0;
  for (int i = tid; i < n; i += blockDim.x) {
    const float v = x[i];
    acc += (double)__fmul_rn(v, v);
  }
  acc = warp_sum_f64(acc);
  if (lane == 0) s_part[warp] = acc;
  __syncthreads();
  if (warp == 0) {
    double t = lane < nwarps ? s_part[lane] : 0.0;
    t = warp_sum_f64(t);
    if (lane == 0) {
      const float mean = (float)(t / (double)n);
      s_scale = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(mean, eps)));
    }
  }
  __syncthreads();
  const float scale = s_scale;
  if constexpr (FAMILY == 1) {
    for (int blk = warp; blk < n / QK_K; blk += nwarps) {
      float v[8];
      const int e0 = blk * QK_K + 8 * lane;
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = __fmul_rn(__fmul_rn(x[e0 + i], scale), w[e0 + i]);
      if (out) {
#pragma unroll
        for (int i = 0; i < 8; ++i) out[e0 + i] = v[i];
      }
      uint32_t lo, hi; int s; float d;
      q8_k_block_warp(v, lane, lo, hi, s, d);
      q8_k_store_planes(planes, 0, n, blk, lane, lo, hi, s, d);
    }
  } else if constexpr (FAMILY == 2) {
    for (int e0 = 4 * tid; e0 < n; e0 += 4 * blockDim.x) {
      float v[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) v[i] = __fmul_rn(__fmul_rn(x[e0 + i], scale), w[e0 + i]);
      if (out) {
#pragma unroll
        for (int i = 0; i < 4; ++i) out[e0 + i] = v[i];
      }
      uint32_t q; __half dh;
      q8_0_block_oct(v, q, dh);
      *reinterpret_cast<uint32_t*>(planes.qs + e0) = q;
      if ((tid & 7) == 0) planes.d[e0 / QK32] = __half2float(dh);
    }
  } else {
    for (int i = tid; i < n; i += blockDim.x) out[i] = __fmul_rn(__fmul_rn(x[i], scale), w[i]);
  }
}

// ---- rotate q and k at `position` with the precomputed cos/sin table row,
// store k and v as f16 into the KV cache rows of that position.
// One thread per rotation pair / per copied element.
__global__ void rope_store_kernel(float* q, const float* k, const float* v, const float* __restrict__ cos_t,
                                  const float* __restrict__ sin_t, const int* pos_dev, int n_head, int n_head_kv,
                                  int head_dim, int rot_dim, int neox, __half* kcache, __half* vcache,
                                  int64_t cache_head_stride /*halves*/) {
  pdl_trigger();
  pdl_wait();
  const int pos = *pos_dev;
  const int pairs = rot_dim / 2;
  const float* ct = cos_t + (int64_t)pos * pairs;
  const float* st = sin_t + (int64_t)pos * pairs;
  const int head = blockIdx.x;
  const int x1_base = neox ? pairs : 1;
  const int stride = neox ? 1 : 2;
  if (head < n_head) {
    float* h = q + (int64_t)head * head_dim;
    for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
      const int d0 = p * stride, d1 = p * stride + x1_base;
      const float x0 = h[d0], x1 = h[d1], c = ct[p], s = st[p];
      h[d0] = __fsub_rn(__fmul_rn(x0, c), __fmul_rn(x1, s));
      h[d1] = __fadd_rn(__fmul_rn(x0, s), __fmul_rn(x1, c));
    }
  } else {
    const int kh = head - n_head;
    const float* h = k + (int64_t)kh * head_dim;
    const float* vv = v + (int64_t)kh * head_dim;
    __half* kd = kcache + (int64_t)kh * cache_head_stride + (int64_t)pos * head_dim;
    __half* vd = vcache + (int64_t)kh * cache_head_stride + (int64_t)pos * head_dim;
    for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
      const int d0 = p * stride, d1 = p * stride + x1_base;
      const float x0 = h[d0], x1 = h[d1], c = ct[p], s = st[p];
      kd[d0] = __float2half_rn(__fsub_rn(__fmul_rn(x0, c), __fmul_rn(x1, s)));
      kd[d1] = __float2half_rn(__fadd_rn(__fmul_rn(x0, s), __fmul_rn(x1, c)));
    }
    for (int d = rot_dim + threadIdx.x; d < head_dim; d += blockDim.x) kd[d] = __float2half_rn(h[d]);
    for (int d = threadIdx.x; d < head_dim; d += blockDim.x) vd[d] = __float2half_rn(vv[d]);
  }
}

// ---- ffn = (gate / (1 + expf(-gate))) * up, quantized for the down projection
template <int FAMILY>
__global__ void __launch_bounds__(256)
swiglu_kernel(const float* __restrict__ gate, const float* __restrict__ up, int n, float* out, ActPlanesMut planes) {
  pdl_trigger();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  if constexpr (FAMILY == 1) {
    // one 256-block per CTA: each of 256 threads one element (the expf dominates), then warp 0 quantizes
    __shared__ float s_v[QK_K];
    const int blk = blockIdx.x;
    const int e = blk * QK_K + threadIdx.x;
    const float g = gate[e];
    const float r = __fmul_rn(__fdiv_rn(g, __fadd_rn(1.0f, expf_exact(-g))), up[e]);
    if (out) out[e] = r;
    s_v[threadIdx.x] = r;
    __syncthreads();
    if (threadIdx.x < 32) {
      float v[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = s_v[8 * lane + i];
      uint32_t lo, hi; int s; float d;
      q8_k_block_warp(v, lane, lo, hi, s, d);
      q8_k_store_planes(planes, 0, n, blk, lane, lo, hi, s, d);
    }
  } else {
    const int e0 = 4 * (blockIdx.x * 128 + threadIdx.x);
    const bool live = e0 < n;
    float v[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    if (live) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float g = gate[e0 + i];
        v[i] = __fmul_rn(__fdiv_rn(g, __fadd_rn(1.0f, expf_exact(-g))), up[e0 + i]);
      }
    }
    if constexpr (FAMILY == 2) {
      uint32_t q; __half dh;
      q8_0_block_oct(v, q, dh);
      if (live) {
        *reinterpret_cast<uint32_t*>(planes.qs + e0) = q;
        if ((threadIdx.x & 7) == 0) planes.d[e0 / QK32] = __half2float(dh);
      }
    }
    if (live && out) {
#pragma unroll
      for (int i = 0; i < 4; ++i) out[e0 + i] = v[i];
    }
  }
}

// ---- embedding row `*token_dev` of a {K, vocab} table -> f32 (same arithmetic
// as the block dequantizers; f32 / f16 tables are copied / widened)
__device__ __forceinline__ uint16_t ld16e(const uint8_t* p) { return (uint16_t)p[0] | ((uint16_t)p[1] << 8); }

// element e of the table row at r
__device__ __forceinline__ float embed_value(int type, const uint8_t* __restrict__ r, int e) {
  float out;
  if (type == T_F32) {
    out = reinterpret_cast<const float*>(r)[e];
  } else if (type == T_F16) {
    out = __half2float(reinterpret_cast<const __half*>(r)[e]);
  } else if (type == T_Q4_K) {
    const uint8_t* b = r + (e / QK_K) * Q4_K_BYTES;
    const int p = e % QK_K, j = p / 32, l = p % 32;
    const float d = h2f(ld16e(b)), mn = h2f(ld16e(b + 2));
    const uint8_t* s = b + 4;
    int sc, m;
    if (j < 4) { sc = s[j] & 63; m = s[j + 4] & 63; }
    else { sc = (s[j + 4] & 0x0f) | ((s[j - 4] >> 6) << 4); m = (s[j + 4] >> 4) | ((s[j] >> 6) << 4); }
    const uint8_t qb = b[16 + 32 * (j >> 1) + l];
    const int q = (j & 1) ? (qb >> 4) : (qb & 0x0f);
    out = __fsub_rn(__fmul_rn(__fmul_rn(d, (float)sc), (float)q), __fmul_rn(mn, (float)m));
  } else if (type == T_Q6_K) {
    const uint8_t* b = r + (e / QK_K) * Q6_K_BYTES;
    const int p = e % QK_K, n = p / 128, pp = p % 128, g = pp / 32, l = pp % 32;
    const uint8_t qlb = b[64 * n + l + 32 * (g & 1)];
    const uint8_t qhb = b[128 + 32 * n + l];
    const int lo = (g & 2) ? (qlb >> 4) : (qlb & 0x0f);
    const int q = (int)(int8_t)(lo | (((qhb >> (2 * g)) & 3) << 4)) - 32;
    const int sc = (int)(int8_t)b[192 + 8 * n + l / 16 + 2 * g];
    out = __fmul_rn(__fmul_rn(h2f(ld16e(b + 208)), (float)sc), (float)q);
  } else if (type == T_Q8_0) {
    const uint8_t* b = r + (e / QK32) * Q8_0_BYTES;
    out = __fmul_rn(h2f(ld16e(b)), (float)(int8_t)b[2 + e % QK32]);
  } else {
    const uint8_t* b = r + (e / QK32) * Q4_0_BYTES;
    const int p = e % QK32;
    const uint8_t qb = b[2 + (p & 15)];
    out = __fmul_rn((float)((p < 16 ? (qb & 0x0f) : (qb >> 4)) - 8), h2f(ld16e(b)));
  }
  return out;
}

__global__ void embed_row_kernel(int type, const uint8_t* __restrict__ table, int64_t row_bytes, const int* token_dev,
                                 float* __restrict__ dst, int K) {
  pdl_trigger();
  pdl_wait();
  const int e = blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= K) return;
  dst[e] = embed_value(type, table + (int64_t)(*token_dev) * row_bytes, e);
}

// ================= token batches (prompt processing) =================
// Activations of a batch of B tokens are kept feature-major: element e of token j at x[e * B + j], the
// layout op_mul_mat reads its right-hand side in and writes its result in (src/emel/kernel/detail.hpp:3356-3571).
// Per token the arithmetic of each kernel is that of its one-token counterpart above.

__global__ void embed_rows_kernel(int type, const uint8_t* __restrict__ table, int64_t row_bytes, const int* __restrict__ tokens,
                                  int B, float* __restrict__ dst, int K) {
  const int e = blockIdx.x * blockDim.x + threadIdx.x, j = blockIdx.y;
  if (e >= K) return;
  dst[(int64_t)e * B + j] = embed_value(type, table + (int64_t)tokens[j] * row_bytes, e);
}

// rms_norm of a token batch in two launches that both fill the machine: (a) f64 sums of squares of one
// feature slice per CTA row (blockIdx.y) for 32 tokens (threadIdx.x), written as partials [slice][token];
// (b) every element scaled, each thread adding its token's partials in slice order.
constexpr int kNormSlices = 16;

__global__ void __launch_bounds__(256)
rms_partial_batch_kernel(const float* __restrict__ x, int K, int B, double* __restrict__ partial) {
  __shared__ double s_part[8][33];
  const int tx = threadIdx.x, ty = threadIdx.y, j = blockIdx.x * 32 + tx;
  const int per = (K + kNormSlices - 1) / kNormSlices;
  const int e0 = blockIdx.y * per, e1 = min(K, e0 + per);
  double acc = 0.0;
  if (j < B) {
    for (int e = e0 + ty; e < e1; e += 8) {
      const float v = x[(int64_t)e * B + j];
      acc += (double)__fmul_rn(v, v);
    }
  }
  s_part[ty][tx] = acc;
  __syncthreads();
  if (ty == 0 && j < B) {
    double t = 0.0;
#pragma unroll
    for (int i = 0; i < 8; ++i) t += s_part[i][tx];
    partial[(int64_t)blockIdx.y * B + j] = t;
  }
}

__global__ void __launch_bounds__(256)
rms_apply_batch_kernel(const float* __restrict__ x, const float* __restrict__ w, const double* __restrict__ partial, float eps,
                       int K, int B, float* __restrict__ out) {
  const int j = blockIdx.x * 32 + threadIdx.x;
  if (j >= B) return;
  double t = 0.0;
#pragma unroll
  for (int i = 0; i < kNormSlices; ++i) t += partial[(int64_t)i * B + j];
  const float mean = (float)(t / (double)K);
  const float scale = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(mean, eps)));
  const int per = (K + gridDim.y - 1) / gridDim.y;
  const int e0 = blockIdx.y * per, e1 = min(K, e0 + per);
  for (int e = e0 + threadIdx.y; e < e1; e += blockDim.y)
    out[(int64_t)e * B + j] = __fmul_rn(__fmul_rn(x[(int64_t)e * B + j], scale), w[e]);
}

// A few columns (a decode step of several sequences): one launch normalises and quantizes.  CTA = one column, 1024
// threads; the squares are summed in f64 (thread partial sums over features t, t + 1024, ..., then warps, then one
// thread in a fixed order), and then warp w takes 256-feature blocks w, w + 32, ...: the lane's 8 elements are
// scaled, multiplied by the weight and quantized to Q8_K like every other activation vector.
__global__ void __launch_bounds__(1024)
rms_norm_quant_cols_kernel(const float* __restrict__ x, const float* __restrict__ w, float eps, int K, int B, ActPlanesMut planes) {
  __shared__ double s_part[32];
  __shared__ float s_scale;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, col = blockIdx.x;
  double ss = 0.0;
#pragma unroll 4
  for (int e = threadIdx.x; e < K; e += 1024) {
    const float v = x[(int64_t)e * B + col];
    ss += (double)__fmul_rn(v, v);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if (lane == 0) s_part[warp] = ss;
  __syncthreads();
  if (threadIdx.x == 0) {
    double t = 0.0;
#pragma unroll
    for (int i = 0; i < 32; ++i) t += s_part[i];
    const float mean = (float)(t / (double)K);
    s_scale = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(mean, eps)));
  }
  __syncthreads();
  const float scale = s_scale;
  for (int blk = warp; blk < K / QK_K; blk += 32) {
    float v[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int e = blk * QK_K + 8 * lane + i;
      v[i] = __fmul_rn(__fmul_rn(x[(int64_t)e * B + col], scale), w[e]);
    }
    uint32_t lo, hi; int bs; float dq;
    q8_k_block_warp(v, lane, lo, hi, bs, dq);
    q8_k_store_planes(planes, col, K, blk, lane, lo, hi, bs, dq);
  }
}

// SwiGLU of a few columns, quantized for the down projection in the same launch: one warp per (256-feature block,
// column), the lane's 8 elements computed from gate and up and quantized to Q8_K
__global__ void __launch_bounds__(256)
swiglu_quant_cols_kernel(const float* __restrict__ gate, const float* __restrict__ up, int K, int B, ActPlanesMut planes) {
  const int lane = threadIdx.x & 31;
  const int item = blockIdx.x * 8 + (threadIdx.x >> 5);
  const int nblk = K / QK_K;
  if (item >= nblk * B) return;
  const int col = item % B, blk = item / B;
  float v[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int64_t o = (int64_t)(blk * QK_K + 8 * lane + i) * B + col;
    const float g = gate[o];
    v[i] = __fmul_rn(__fdiv_rn(g, __fadd_rn(1.0f, expf_exact(-g))), up[o]);
  }
  uint32_t lo, hi; int bs; float dq;
  q8_k_block_warp(v, lane, lo, hi, bs, dq);
  q8_k_store_planes(planes, col, K, blk, lane, lo, hi, bs, dq);
}

// thread = (token j fastest, rotation pair or copied element, head).  Query heads are rotated in place.  K / V heads
// go to the f16 cache: the inputs are feature-major (tokens along the lanes) and a cache row is one token's head_dim
// halves, so storing straight from the registers would put 2 bytes per lane into 32 different rows; with `rows`
// a 32-token tile of the rotated K head and of the V head is put together in shared memory (2 x 32 x (head_dim + 8)
// halves) and each warp then writes whole rows, 8 bytes per lane.
__global__ void __launch_bounds__(256)
rope_store_batch_kernel(float* q, const float* __restrict__ k, const float* __restrict__ v, const float* __restrict__ cos_t,
                        const float* __restrict__ sin_t, int pos0, int B, int n_head, int n_head_kv, int head_dim, int rot_dim,
                        int neox, __half* kcache, __half* vcache, int64_t cache_head_stride, int rows) {
  extern __shared__ __align__(16) __half kv_tile[];
  const int j0 = blockIdx.x * 32, j = j0 + threadIdx.x;
  const bool live = j < B;
  const int head = blockIdx.y, pos = pos0 + (live ? j : 0), pairs = rot_dim / 2;
  const float* ct = cos_t + (int64_t)pos * pairs;
  const float* st = sin_t + (int64_t)pos * pairs;
  const int x1_base = neox ? pairs : 1, stride = neox ? 1 : 2;
  if (head < n_head) {
    if (!live) return;
    float* h = q + (int64_t)head * head_dim * B + j;
    for (int p = threadIdx.y; p < pairs; p += blockDim.y) {
      const int64_t d0 = (int64_t)(p * stride) * B, d1 = (int64_t)(p * stride + x1_base) * B;
      const float x0 = h[d0], x1 = h[d1], c = ct[p], s = st[p];
      h[d0] = __fsub_rn(__fmul_rn(x0, c), __fmul_rn(x1, s));
      h[d1] = __fadd_rn(__fmul_rn(x0, s), __fmul_rn(x1, c));
    }
    return;
  }
  const int kh = head - n_head;
  const int row = head_dim + 8;
  // destination of this thread's values: its token's cache rows, or its token's rows of the tile
  __half* kd = rows ? kv_tile + threadIdx.x * row : kcache + (int64_t)kh * cache_head_stride + (int64_t)pos * head_dim;
  __half* vd = rows ? kv_tile + (32 + threadIdx.x) * row : vcache + (int64_t)kh * cache_head_stride + (int64_t)pos * head_dim;
  if (live) {
    const float* h = k + (int64_t)kh * head_dim * B + j;
    const float* vv = v + (int64_t)kh * head_dim * B + j;
    for (int p = threadIdx.y; p < pairs; p += blockDim.y) {
      const int d0 = p * stride, d1 = p * stride + x1_base;
      const float x0 = h[(int64_t)d0 * B], x1 = h[(int64_t)d1 * B], c = ct[p], s = st[p];
      kd[d0] = __float2half_rn(__fsub_rn(__fmul_rn(x0, c), __fmul_rn(x1, s)));
      kd[d1] = __float2half_rn(__fadd_rn(__fmul_rn(x0, s), __fmul_rn(x1, c)));
    }
    for (int d = rot_dim + threadIdx.y; d < head_dim; d += blockDim.y) kd[d] = __float2half_rn(h[(int64_t)d * B]);
    for (int d = threadIdx.y; d < head_dim; d += blockDim.y) vd[d] = __float2half_rn(vv[(int64_t)d * B]);
  }
  if (!rows) return;
  __syncthreads();
  for (int t = threadIdx.y; t < 32 && j0 + t < B; t += blockDim.y) {
    const int64_t off = (int64_t)kh * cache_head_stride + (int64_t)(pos0 + j0 + t) * head_dim;
    for (int d = 4 * threadIdx.x; d < head_dim; d += 128) {
      *reinterpret_cast<uint2*>(kcache + off + d) = *reinterpret_cast<const uint2*>(kv_tile + t * row + d);
      *reinterpret_cast<uint2*>(vcache + off + d) = *reinterpret_cast<const uint2*>(kv_tile + (32 + t) * row + d);
    }
  }
}

// one decode step of several sequences: column j is sequence j at its own position.  Thread = (sequence j fastest,
// slot, head): a slot is one rotation pair or, past the rotated dimensions, two copied elements; heads are the
// query heads, then the K heads, then the V heads (two elements per slot, no rotation)
__global__ void __launch_bounds__(256)
rope_store_seqs_kernel(const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v,
                       const float* __restrict__ cos_t, const float* __restrict__ sin_t, const int* __restrict__ positions, int B,
                       int n_head, int n_head_kv, int head_dim, int rot_dim, int neox, float* __restrict__ q_out, __half* kcache,
                       __half* vcache, int64_t seq_stride, int64_t cache_head_stride) {
  const int half = head_dim / 2, pairs = rot_dim / 2;
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t total = (int64_t)(n_head + 2 * n_head_kv) * half * B;
  if (idx >= total) return;
  const int j = (int)(idx % B);
  const int slot = (int)((idx / B) % half);
  const int head = (int)(idx / ((int64_t)B * half));
  const int pos = positions[j];
  int d0, d1;
  float c = 1.0f, sn = 0.0f;
  const bool is_v = head >= n_head + n_head_kv;
  const bool rotate = !is_v && slot < pairs;
  if (rotate) {
    d0 = neox ? slot : 2 * slot;
    d1 = neox ? slot + pairs : 2 * slot + 1;
    c = cos_t[(int64_t)pos * pairs + slot];
    sn = sin_t[(int64_t)pos * pairs + slot];
  } else if (is_v) {
    d0 = 2 * slot;
    d1 = 2 * slot + 1;
  } else {
    d0 = rot_dim + 2 * (slot - pairs);
    d1 = d0 + 1;
  }
  const float* src = head < n_head ? q + (int64_t)head * head_dim * B
                                   : (is_v ? v + (int64_t)(head - n_head - n_head_kv) * head_dim * B : k + (int64_t)(head - n_head) * head_dim * B);
  const float x0 = src[(int64_t)d0 * B + j], x1 = src[(int64_t)d1 * B + j];
  float o0 = x0, o1 = x1;
  if (rotate) {
    o0 = __fsub_rn(__fmul_rn(x0, c), __fmul_rn(x1, sn));
    o1 = __fadd_rn(__fmul_rn(x0, sn), __fmul_rn(x1, c));
  }
  if (head < n_head) {
    float* o = q_out + ((int64_t)j * n_head + head) * head_dim;
    o[d0] = o0;
    o[d1] = o1;
  } else {
    const int kh = is_v ? head - n_head - n_head_kv : head - n_head;
    __half* dst = (is_v ? vcache : kcache) + (int64_t)j * seq_stride + (int64_t)kh * cache_head_stride + (int64_t)pos * head_dim;
    dst[d0] = __float2half_rn(o0);
    dst[d1] = __float2half_rn(o1);
  }
}

__global__ void batch_begin_kernel(int* state, int stride, int B) {
  const int j = threadIdx.x;
  if (j < B) state[2 * stride + j] = state[stride + j] + 1;
  if (j == 0) state[3 * stride] = 0;
}

__global__ void batch_advance_kernel(int* state, int stride, int B, const int* __restrict__ idx, int* out) {
  const int j = threadIdx.x;
  const int step = state[3 * stride];
  __syncthreads();
  if (j < B) {
    state[j] = idx[j];
    state[stride + j] += 1;
    state[2 * stride + j] += 1;
    out[(int64_t)step * B + j] = idx[j];
  }
  if (j == 0) state[3 * stride] = step + 1;
}

// argmax per column of x {rows, B} (column index fastest): CTA b scans a row range for every column, thread t
// column t % B; then one CTA per launch folds the candidates.  Highest value, lowest row on ties; a NaN never
// replaces a candidate (the reference's `>` comparison)
__device__ __forceinline__ bool argmax_better(float v, int r, float bv, int br) { return br < 0 || v > bv || (v == bv && r < br); }

__global__ void __launch_bounds__(256) argmax_columns_part_kernel(const float* __restrict__ x, int rows, int B, float* part_val, int* part_idx) {
  __shared__ float s_v[256];
  __shared__ int s_i[256];
  const int lanes = 256 / B;            // row lanes per column
  const int col = threadIdx.x % B, rl = threadIdx.x / B;
  const int per = (rows + gridDim.x - 1) / gridDim.x;
  const int r0 = blockIdx.x * per, r1 = min(rows, r0 + per);
  float bv = 0.0f;
  int bi = -1;
  if (rl < lanes)
    for (int r = r0 + rl; r < r1; r += lanes) {
      const float v = x[(int64_t)r * B + col];
      if (argmax_better(v, r, bv, bi)) { bv = v; bi = r; }
    }
  s_v[threadIdx.x] = bv;
  s_i[threadIdx.x] = bi;
  __syncthreads();
  if (threadIdx.x < B) {
    for (int l = 1; l < lanes; ++l) {
      const float v = s_v[l * B + col];
      const int r = s_i[l * B + col];
      if (r >= 0 && argmax_better(v, r, bv, bi)) { bv = v; bi = r; }
    }
    part_val[blockIdx.x * B + col] = bv;
    part_idx[blockIdx.x * B + col] = bi;
  }
}

__global__ void argmax_columns_finish_kernel(const float* part_val, const int* part_idx, int parts, int B, int* out_idx) {
  const int col = threadIdx.x;
  if (col >= B) return;
  float bv = 0.0f;
  int bi = -1;
  for (int p = 0; p < parts; ++p) {
    const float v = part_val[p * B + col];
    const int r = part_idx[p * B + col];
    if (r >= 0 && argmax_better(v, r, bv, bi)) { bv = v; bi = r; }
  }
  out_idx[col] = bi < 0 ? 0 : bi;
}

__global__ void add_inplace_kernel(float* __restrict__ acc, const float* __restrict__ y, int64_t n) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) acc[i] = __fadd_rn(acc[i], y[i]);
}

// ---- step bookkeeping on the device so a captured graph can run token after
// token without the host: state = {token, position, kv_tokens, step}
__global__ void step_begin_kernel(int* state, int token, int position) {
  state[0] = token;
  state[1] = position;
  state[2] = position + 1;
  state[3] = 0;
}
__global__ void step_advance_kernel(int* state, const int* best_idx, int* tokens_out) {
  pdl_trigger();
  pdl_wait();
  const int t = *best_idx;
  tokens_out[state[3]] = t;
  state[0] = t;
  state[1] += 1;
  state[2] += 1;
  state[3] += 1;
}

}  // namespace

cudaError_t launch_rms_norm(const float* x, const float* w, float eps, int n, float* out, int family, ActPlanesMut planes,
                            cudaStream_t st) {
  const int threads = n >= 4096 ? 1024 : (n >= 1024 ? 256 : 128);
  if (family == 1) EMELB_LAUNCH(rms_norm_kernel<1>, 1, threads, 0, st, x, w, eps, n, out, planes);
  else if (family == 2) EMELB_LAUNCH(rms_norm_kernel<2>, 1, threads, 0, st, x, w, eps, n, out, planes);
  else EMELB_LAUNCH(rms_norm_kernel<0>, 1, threads, 0, st, x, w, eps, n, out, planes);
  return cudaGetLastError();
}

cudaError_t launch_rope_store(float* q, const float* k, const float* v, const float* cos_t, const float* sin_t,
                              const int* pos_dev, int n_head, int n_head_kv, int head_dim, int rot_dim, int neox,
                              __half* kcache, __half* vcache, int64_t cache_head_stride, cudaStream_t st) {
  EMELB_LAUNCH(rope_store_kernel, n_head + n_head_kv, 64, 0, st, q, k, v, cos_t, sin_t, pos_dev, n_head, n_head_kv, head_dim,
                                                       rot_dim, neox, kcache, vcache, cache_head_stride);
  return cudaGetLastError();
}

// ---- op_rms_norm as an op of its own (src/emel/kernel/detail.hpp:4567-4602): per row, f64 sum of the f32
// squares, scale = 1 / sqrt(mean + eps), out = x * scale (no weight vector: that is the generator's rms_norm)
__global__ void __launch_bounds__(256) rms_norm_rows_kernel(const StridedF32 src, const StridedF32 dst, float eps) {
  __shared__ double s_part[8];
  const int64_t row = blockIdx.x;
  const int64_t i1 = row % src.ne[1], i2 = (row / src.ne[1]) % src.ne[2], i3 = row / (src.ne[1] * src.ne[2]);
  const char* srow = src.base + i1 * src.nb[1] + i2 * src.nb[2] + i3 * src.nb[3];
  char* drow = dst.base + i1 * dst.nb[1] + i2 * dst.nb[2] + i3 * dst.nb[3];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  double ss = 0.0;
  for (int64_t i0 = threadIdx.x; i0 < src.ne[0]; i0 += 256) {
    const float v = *reinterpret_cast<const float*>(srow + i0 * src.nb[0]);
    ss += (double)__fmul_rn(v, v);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if (lane == 0) s_part[warp] = ss;
  __syncthreads();
  double total = 0.0;
#pragma unroll
  for (int w = 0; w < 8; ++w) total += s_part[w];
  const float mean = (float)(total / (double)src.ne[0]);
  const float scale = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(mean, eps)));
  for (int64_t i0 = threadIdx.x; i0 < src.ne[0]; i0 += 256) {
    const float v = *reinterpret_cast<const float*>(srow + i0 * src.nb[0]);
    *reinterpret_cast<float*>(drow + i0 * dst.nb[0]) = __fmul_rn(v, scale);
  }
}

// ---- op_rope as an op of its own (run_rope_as, src/emel/kernel/detail.hpp:4706-4765): one thread per row;
// theta starts at the row's position and is multiplied by theta_scale pair after pair (the reference's float
// recurrence), cos / sin of theta * freq_scale, times attn_factor; dims past n_dims are copied
__global__ void __launch_bounds__(128) rope_rows_kernel(const StridedF32 src, const StridedF32 dst, const char* pos_base,
                                                        int64_t pos_stride, int n_dims, int neox, float theta_scale,
                                                        float freq_scale, float attn_factor) {
  const int64_t rows = src.ne[1] * src.ne[2] * src.ne[3];
  const int64_t row = (int64_t)blockIdx.x * 128 + threadIdx.x;
  if (row >= rows) return;
  const int64_t i1 = row % src.ne[1], i2 = (row / src.ne[1]) % src.ne[2], i3 = row / (src.ne[1] * src.ne[2]);
  const char* srow = src.base + i1 * src.nb[1] + i2 * src.nb[2] + i3 * src.nb[3];
  char* drow = dst.base + i1 * dst.nb[1] + i2 * dst.nb[2] + i3 * dst.nb[3];
  const int half = n_dims / 2;
  float theta = (float)*reinterpret_cast<const int32_t*>(pos_base + i2 * pos_stride);
  for (int pair = 0; pair < half; ++pair, theta = __fmul_rn(theta, theta_scale)) {
    const float rotated = __fmul_rn(theta, freq_scale);
    const float cs = __fmul_rn(cosf(rotated), attn_factor), sn = __fmul_rn(sinf(rotated), attn_factor);
    const int64_t a = neox ? pair : 2 * pair, b = neox ? pair + half : 2 * pair + 1;
    const float x0 = *reinterpret_cast<const float*>(srow + a * src.nb[0]);
    const float x1 = *reinterpret_cast<const float*>(srow + b * src.nb[0]);
    *reinterpret_cast<float*>(drow + a * dst.nb[0]) = __fsub_rn(__fmul_rn(x0, cs), __fmul_rn(x1, sn));
    *reinterpret_cast<float*>(drow + b * dst.nb[0]) = __fadd_rn(__fmul_rn(x0, sn), __fmul_rn(x1, cs));
  }
  for (int64_t i0 = n_dims; i0 < src.ne[0]; ++i0)
    *reinterpret_cast<float*>(drow + i0 * dst.nb[0]) = *reinterpret_cast<const float*>(srow + i0 * src.nb[0]);
}

cudaError_t launch_rms_norm_rows(const StridedF32& src, const StridedF32& dst, float eps, cudaStream_t st) {
  const int64_t rows = src.ne[1] * src.ne[2] * src.ne[3];
  rms_norm_rows_kernel<<<(unsigned)rows, 256, 0, st>>>(src, dst, eps);
  return cudaGetLastError();
}

cudaError_t launch_rope_rows(const StridedF32& src, const StridedF32& dst, const char* pos_base, int64_t pos_stride, int n_dims,
                             int neox, float theta_scale, float freq_scale, float attn_factor, cudaStream_t st) {
  const int64_t rows = src.ne[1] * src.ne[2] * src.ne[3];
  rope_rows_kernel<<<(unsigned)((rows + 127) / 128), 128, 0, st>>>(src, dst, pos_base, pos_stride, n_dims, neox, theta_scale,
                                                                   freq_scale, attn_factor);
  return cudaGetLastError();
}

// the SwiGLU of this rank's interval of the ffn vector: one 256-block per CTA, quantized to Q8_K once and written
// into every rank's planes of the joined vector
__global__ void __launch_bounds__(256) swiglu_join_kernel(const float* __restrict__ gate, const float* __restrict__ up, const JoinOut* __restrict__ join_dev) {
  pdl_trigger();
  const JoinOut jo = *join_dev;   // a constant of the session: fetched before the wait for the preceding kernel
  pdl_wait();
  __shared__ float s_v[QK_K];
  const int lane = threadIdx.x & 31;
  const int e = blockIdx.x * QK_K + threadIdx.x;
  const float g = gate[e];
  s_v[threadIdx.x] = __fmul_rn(__fdiv_rn(g, __fadd_rn(1.0f, expf_exact(-g))), up[e]);
  __syncthreads();
  if (threadIdx.x < 32) {
    float v[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = s_v[8 * lane + i];
    uint32_t lo, hi; int bs; float d;
    q8_k_block_warp(v, lane, lo, hi, bs, d);
    join_store_q8_k_block(jo, jo.first_block + blockIdx.x, lane, lo, hi, bs, d);
  }
  join_publish(jo, gridDim.x);
}

cudaError_t launch_swiglu_join(const float* gate, const float* up, int n, const JoinOut* join_dev, cudaStream_t st) {
  if (n % QK_K != 0 || !join_dev) return cudaErrorInvalidValue;
  EMELB_LAUNCH(swiglu_join_kernel, n / QK_K, 256, 0, st, gate, up, join_dev);
  return cudaGetLastError();
}

cudaError_t launch_swiglu(const float* gate, const float* up, int n, float* out, int family, ActPlanesMut planes,
                          cudaStream_t st) {
  if (family == 1) EMELB_LAUNCH(swiglu_kernel<1>, n / QK_K, 256, 0, st, gate, up, n, out, planes);
  else if (family == 2) EMELB_LAUNCH(swiglu_kernel<2>, (n / 4 + 127) / 128, 128, 0, st, gate, up, n, out, planes);
  else EMELB_LAUNCH(swiglu_kernel<0>, (n / 4 + 127) / 128, 128, 0, st, gate, up, n, out, planes);
  return cudaGetLastError();
}

cudaError_t launch_embed_row(int type, const uint8_t* table, int64_t row_bytes, const int* token_dev, float* dst, int K,
                             cudaStream_t st) {
  EMELB_LAUNCH(embed_row_kernel, (K + 255) / 256, 256, 0, st, type, table, row_bytes, token_dev, dst, K);
  return cudaGetLastError();
}

cudaError_t launch_embed_rows(int type, const uint8_t* table, int64_t row_bytes, const int* tokens_dev, int B, float* dst,
                              int K, cudaStream_t st) {
  embed_rows_kernel<<<dim3((K + 255) / 256, B), 256, 0, st>>>(type, table, row_bytes, tokens_dev, B, dst, K);
  return cudaGetLastError();
}

cudaError_t launch_rms_norm_batch(const float* x, const float* w, float eps, int K, int B, float* out, double* partial,
                                  cudaStream_t st) {
  const int tiles = (B + 31) / 32;
  rms_partial_batch_kernel<<<dim3(tiles, kNormSlices), dim3(32, 8), 0, st>>>(x, K, B, partial);
  int slices = K / 64 > 0 ? K / 64 : 1;        // 64 features x 32 tokens per CTA
  if (slices > 1024) slices = 1024;
  rms_apply_batch_kernel<<<dim3(tiles, slices), dim3(32, 8), 0, st>>>(x, w, partial, eps, K, B, out);
  return cudaGetLastError();
}

int rms_norm_batch_partials(int B) { return kNormSlices * B; }

cudaError_t launch_rope_store_batch(float* q, const float* k, const float* v, const float* cos_t, const float* sin_t, int pos0,
                                    int B, int n_head, int n_head_kv, int head_dim, int rot_dim, int neox, __half* kcache,
                                    __half* vcache, int64_t cache_head_stride, cudaStream_t st) {
  // cache rows written as rows where the layout allows 8-byte stores
  const size_t tile_bytes = 2 * 32 * (size_t)(head_dim + 8) * sizeof(__half);
  const bool rows = head_dim % 4 == 0 && cache_head_stride % 4 == 0 && tile_bytes <= 48 * 1024 &&
                    reinterpret_cast<uintptr_t>(kcache) % 8 == 0 && reinterpret_cast<uintptr_t>(vcache) % 8 == 0;
  rope_store_batch_kernel<<<dim3((B + 31) / 32, n_head + n_head_kv), dim3(32, 8), rows ? tile_bytes : 0, st>>>(
      q, k, v, cos_t, sin_t, pos0, B, n_head, n_head_kv, head_dim, rot_dim, neox, kcache, vcache, cache_head_stride, rows ? 1 : 0);
  return cudaGetLastError();
}

cudaError_t launch_rope_store_seqs(const float* q, const float* k, const float* v, const float* cos_t, const float* sin_t,
                                   const int* positions, int B, int n_head, int n_head_kv, int head_dim, int rot_dim, int neox,
                                   float* q_out, __half* kcache, __half* vcache, int64_t seq_stride, int64_t cache_head_stride,
                                   cudaStream_t st) {
  if (head_dim % 2 != 0 || rot_dim % 2 != 0) return cudaErrorInvalidValue;
  const int64_t total = (int64_t)(n_head + 2 * n_head_kv) * (head_dim / 2) * B;
  rope_store_seqs_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(q, k, v, cos_t, sin_t, positions, B, n_head, n_head_kv,
                                                                         head_dim, rot_dim, neox, q_out, kcache, vcache, seq_stride,
                                                                         cache_head_stride);
  return cudaGetLastError();
}

cudaError_t launch_swiglu_quant_cols(const float* gate, const float* up, int K, int B, ActPlanesMut planes, cudaStream_t st) {
  if (K % QK_K != 0 || B < 1) return cudaErrorInvalidValue;
  const int items = K / QK_K * B;
  swiglu_quant_cols_kernel<<<(items + 7) / 8, 256, 0, st>>>(gate, up, K, B, planes);
  return cudaGetLastError();
}

cudaError_t launch_rms_norm_quant_cols(const float* x, const float* w, float eps, int K, int B, ActPlanesMut planes, cudaStream_t st) {
  if (K % QK_K != 0 || B < 1) return cudaErrorInvalidValue;
  rms_norm_quant_cols_kernel<<<B, 1024, 0, st>>>(x, w, eps, K, B, planes);
  return cudaGetLastError();
}

cudaError_t launch_batch_begin(int* state, int stride, int B, cudaStream_t st) {
  if (B < 1 || B > 256) return cudaErrorInvalidValue;
  batch_begin_kernel<<<1, 256, 0, st>>>(state, stride, B);
  return cudaGetLastError();
}

cudaError_t launch_batch_advance(int* state, int stride, int B, const int* idx, int* out, cudaStream_t st) {
  if (B < 1 || B > 256) return cudaErrorInvalidValue;
  batch_advance_kernel<<<1, 256, 0, st>>>(state, stride, B, idx, out);
  return cudaGetLastError();
}

cudaError_t launch_argmax_columns(const float* x, int rows, int B, float* part_val, int* part_idx, int* out_idx, cudaStream_t st) {
  if (B < 1 || B > 256 || rows < 1) return cudaErrorInvalidValue;
  const int parts = rows < kArgmaxColumnParts ? rows : kArgmaxColumnParts;
  argmax_columns_part_kernel<<<parts, 256, 0, st>>>(x, rows, B, part_val, part_idx);
  argmax_columns_finish_kernel<<<1, 256, 0, st>>>(part_val, part_idx, parts, B, out_idx);
  return cudaGetLastError();
}

cudaError_t launch_add_inplace(float* acc, const float* y, int64_t n, cudaStream_t st) {
  add_inplace_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(acc, y, n);
  return cudaGetLastError();
}

// sharded greedy head: this rank's winner as {value bits, global row}, then the
// winner over all ranks with the reference's tie rule (highest value, lowest row;
// src/emel/kernel/detail.hpp:3720-3723)
__global__ void argmax_pair_store_kernel(const float* best_val, const int* best_idx, int row_offset, int* pair) {
  pair[0] = __float_as_int(*best_val);
  pair[1] = *best_idx + row_offset;
}

__global__ void argmax_pair_finish_kernel(const int* pairs, int n, float* out_val, int* out_idx) {
  float bv = __int_as_float(pairs[0]);
  int bi = pairs[1];
  for (int i = 1; i < n; ++i) {
    const float v = __int_as_float(pairs[4 * i]);   // one 16-byte record per rank
    const int r = pairs[4 * i + 1];
    if (v > bv || (v == bv && r < bi)) { bv = v; bi = r; }
  }
  *out_val = bv;
  *out_idx = bi;
}

cudaError_t launch_argmax_pair_store(const float* best_val, const int* best_idx, int row_offset, int* pair, cudaStream_t st) {
  argmax_pair_store_kernel<<<1, 1, 0, st>>>(best_val, best_idx, row_offset, pair);
  return cudaGetLastError();
}

cudaError_t launch_argmax_pair_finish(const int* pairs, int n, float* out_val, int* out_idx, cudaStream_t st) {
  argmax_pair_finish_kernel<<<1, 1, 0, st>>>(pairs, n, out_val, out_idx);
  return cudaGetLastError();
}

cudaError_t launch_step_begin(int* state, int token, int position, cudaStream_t st) {
  step_begin_kernel<<<1, 1, 0, st>>>(state, token, position);
  return cudaGetLastError();
}

cudaError_t launch_step_advance(int* state, const int* best_idx, int* tokens_out, cudaStream_t st) {
  EMELB_LAUNCH(step_advance_kernel, 1, 1, 0, st, state, best_idx, tokens_out);
  return cudaGetLastError();
}

}  // namespace emelb
