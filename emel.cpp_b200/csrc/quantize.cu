// Activation quantizers and block dequantizers — the bit-exact kernels.
// This file is compiled with -fmad=false and uses the IEEE round-to-nearest
// intrinsics for every division, so each float operation rounds exactly as the
// reference's C++ does when built without contraction:
//   quantize_row_q8_k_strided   src/emel/kernel/detail.hpp:826-867
//   quantize_row_q8_0_strided   src/emel/kernel/detail.hpp:804-824
//   dequantize_row_q4_k/q6_k/q8_0/q4_0   :523-552, 592-629, 679-690, 487-502
#include "quant_device.cuh"

namespace emelb {

namespace {

// One warp per (256-block, column).
template <bool BLOCKS>
__global__ void __launch_bounds__(128)
quantize_q8_k_kernel(const float* __restrict__ x, int n, int K, ActPlanesMut planes, uint8_t* blocks, int64_t row_bytes) {
  pdl_trigger();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int blk = blockIdx.x * 4 + (threadIdx.x >> 5);
  const int col = blockIdx.y;
  if (blk >= K / QK_K) return;
  const float* src = x + ((int64_t)blk * QK_K + 8 * lane) * n + col;
  float v[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) v[i] = src[(int64_t)i * n];
  uint32_t lo, hi;
  int s;
  float d;
  q8_k_block_warp(v, lane, lo, hi, s, d);
  if constexpr (BLOCKS) {
    // reference layout: f32 d, i8 qs[256], i16 bsums[16]; 4-byte aligned only
    uint8_t* b = blocks + (int64_t)col * row_bytes + (int64_t)blk * Q8_K_BYTES;
    uint32_t* qw = reinterpret_cast<uint32_t*>(b + 4 + 8 * lane);
    qw[0] = lo; qw[1] = hi;
    if ((lane & 1) == 0) *reinterpret_cast<int16_t*>(b + 260 + 2 * (lane >> 1)) = (int16_t)s;
    if (lane == 0) *reinterpret_cast<float*>(b) = d;
  } else {
    q8_k_store_planes(planes, col, K, blk, lane, lo, hi, s, d);
  }
}

// Many columns (a prompt batch): one CTA per (256-block, 32 columns).  The input is feature-major, {K, n}: the 256
// elements of a column's block lie n floats apart, so the kernel above fetches a 32-byte sector for every float.  Here
// the f32 tile is read with the columns along the lanes (every load a full line), transposed through shared memory, and
// the warps then quantize one column each exactly as above.
constexpr int kQTileCols = 32, kQTileRow = QK_K + 4;   // rows stay 16-byte aligned for the float4 reads

__global__ void __launch_bounds__(256)
quantize_q8_k_cols_kernel(const float* __restrict__ x, int n, int ncols, int K, ActPlanesMut planes) {
  __shared__ __align__(16) float tile[kQTileCols][kQTileRow];
  pdl_trigger();
  pdl_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int blk = blockIdx.x, c0 = blockIdx.y * kQTileCols;
  const int col = min(c0 + lane, ncols - 1);                // lanes past the edge repeat the last column; never stored
  const float* src = x + (int64_t)blk * QK_K * n + col;
#pragma unroll 8
  for (int j = 0; j < QK_K / 8; ++j) {
    const int k = warp + 8 * j;
    tile[lane][k] = src[(int64_t)k * n];
  }
  __syncthreads();
  for (int c = warp; c < kQTileCols && c0 + c < ncols; c += 8) {
    const float4 a = *reinterpret_cast<const float4*>(&tile[c][8 * lane]);
    const float4 b = *reinterpret_cast<const float4*>(&tile[c][8 * lane + 4]);
    float v[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
    uint32_t lo, hi;
    int s;
    float d;
    q8_k_block_warp(v, lane, lo, hi, s, d);
    q8_k_store_planes(planes, c0 + c, K, blk, lane, lo, hi, s, d);
  }
}

// Eight lanes per 32-block, four elements per lane
template <bool BLOCKS>
__global__ void __launch_bounds__(128)
quantize_q8_0_kernel(const float* __restrict__ x, int n, int K, ActPlanesMut planes, uint8_t* blocks, int64_t row_bytes) {
  pdl_trigger();
  pdl_wait();
  const int sub = threadIdx.x & 7;
  const int blk = blockIdx.x * 16 + (threadIdx.x >> 3);
  const int col = blockIdx.y;
  const bool live = blk < K / QK32;
  const int cb = live ? blk : 0;
  const float* src = x + ((int64_t)cb * QK32 + 4 * sub) * n + col;
  float v[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) v[i] = src[(int64_t)i * n];
  uint32_t w;
  __half dh;
  q8_0_block_oct(v, w, dh);
  if (!live) return;
  if constexpr (BLOCKS) {
    uint8_t* b = blocks + (int64_t)col * row_bytes + (int64_t)blk * Q8_0_BYTES;
    uint16_t* qh = reinterpret_cast<uint16_t*>(b + 2 + 4 * sub);  // 2-byte aligned payload
    qh[0] = (uint16_t)(w & 0xffffu);
    qh[1] = (uint16_t)(w >> 16);
    if (sub == 0) *reinterpret_cast<uint16_t*>(b) = __half_as_ushort(dh);
  } else {
    *reinterpret_cast<uint32_t*>(planes.qs + (int64_t)col * K + (int64_t)blk * QK32 + 4 * sub) = w;
    if (sub == 0) planes.d[(int64_t)col * (K / QK32) + blk] = __half2float(dh);
  }
}

__global__ void blocks_to_planes_q8_k_kernel(const uint8_t* __restrict__ blocks, int nblk, ActPlanesMut out) {
  const int blk = blockIdx.x;
  const uint8_t* b = blocks + (int64_t)blk * Q8_K_BYTES;
  const int t = threadIdx.x;  // 64 threads
  if (blk >= nblk) return;
  reinterpret_cast<uint32_t*>(out.qs + (int64_t)blk * QK_K)[t] = *reinterpret_cast<const uint32_t*>(b + 4 + 4 * t);
  if (t < 16) out.bsums[blk * 16 + t] = *reinterpret_cast<const int16_t*>(b + 260 + 2 * t);
  if (t == 0) out.d[blk] = *reinterpret_cast<const float*>(b);
}

__global__ void blocks_to_planes_q8_0_kernel(const uint8_t* __restrict__ blocks, int nblk, ActPlanesMut out) {
  const int blk = blockIdx.x * 8 + (threadIdx.x >> 4);
  const int t = threadIdx.x & 15;  // 16 threads per block, 2 bytes each
  if (blk >= nblk) return;
  const uint8_t* b = blocks + (int64_t)blk * Q8_0_BYTES;
  reinterpret_cast<uint16_t*>(out.qs + (int64_t)blk * QK32)[t] = *reinterpret_cast<const uint16_t*>(b + 2 + 2 * t);
  if (t == 0) out.d[blk] = h2f(*reinterpret_cast<const uint16_t*>(b));
}

// ---- dequantizers: one thread per output element, scalar loads (rows of
// embedding tables and parity checks; not a bandwidth path)
__device__ __forceinline__ uint16_t ld16u(const uint8_t* p) { return (uint16_t)p[0] | ((uint16_t)p[1] << 8); }

template <int T>
__global__ void dequantize_kernel(const uint8_t* __restrict__ src, int64_t src_row_bytes, float* __restrict__ dst,
                                  int64_t dst_row_elems, int K, int M) {
  const int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int row = blockIdx.y;
  if (e >= K || row >= M) return;
  const uint8_t* r = src + (int64_t)row * src_row_bytes;
  float out;
  if constexpr (T == T_Q4_K) {
    const uint8_t* b = r + (e / QK_K) * Q4_K_BYTES;
    const int p = (int)(e % QK_K), j = p / 32, l = p % 32;
    const float d = h2f(ld16u(b)), mn = h2f(ld16u(b + 2));
    const uint8_t* s = b + 4;
    int sc, m;
    if (j < 4) { sc = s[j] & 63; m = s[j + 4] & 63; }
    else { sc = (s[j + 4] & 0x0f) | ((s[j - 4] >> 6) << 4); m = (s[j + 4] >> 4) | ((s[j] >> 6) << 4); }
    const uint8_t qb = b[16 + 32 * (j >> 1) + l];
    const int q = (j & 1) ? (qb >> 4) : (qb & 0x0f);
    const float d1 = __fmul_rn(d, (float)sc), m1 = __fmul_rn(mn, (float)m);
    out = __fsub_rn(__fmul_rn(d1, (float)q), m1);
  } else if constexpr (T == T_Q6_K) {
    const uint8_t* b = r + (e / QK_K) * Q6_K_BYTES;
    const int p = (int)(e % QK_K), n = p / 128, pp = p % 128, g = pp / 32, l = pp % 32;
    const uint8_t qlb = b[64 * n + l + 32 * (g & 1)];
    const uint8_t qhb = b[128 + 32 * n + l];
    const int lo = (g & 2) ? (qlb >> 4) : (qlb & 0x0f);
    const int q = (int)(int8_t)(lo | (((qhb >> (2 * g)) & 3) << 4)) - 32;
    const int sc = (int)(int8_t)b[192 + 8 * n + l / 16 + 2 * g];
    const float d = h2f(ld16u(b + 208));
    out = __fmul_rn(__fmul_rn(d, (float)sc), (float)q);
  } else if constexpr (T == T_Q8_0) {
    const uint8_t* b = r + (e / QK32) * Q8_0_BYTES;
    out = __fmul_rn(h2f(ld16u(b)), (float)(int8_t)b[2 + e % QK32]);
  } else {
    const uint8_t* b = r + (e / QK32) * Q4_0_BYTES;
    const int p = (int)(e % QK32);
    const uint8_t qb = b[2 + (p & 15)];
    const int q = (p < 16 ? (qb & 0x0f) : (qb >> 4)) - 8;
    out = __fmul_rn((float)q, h2f(ld16u(b)));
  }
  dst[(int64_t)row * dst_row_elems + e] = out;
}

}  // namespace

cudaError_t launch_quantize_q8_k_planes(const float* x, int n, int ncols, int K, ActPlanesMut out, cudaStream_t st) {
  if (ncols >= 16) {
    const dim3 tiles(K / QK_K, (ncols + kQTileCols - 1) / kQTileCols);
    EMELB_LAUNCH(quantize_q8_k_cols_kernel, tiles, 256, 0, st, x, n, ncols, K, out);
    return cudaGetLastError();
  }
  const dim3 grid((K / QK_K + 3) / 4, ncols);
  EMELB_LAUNCH(quantize_q8_k_kernel<false>, grid, 128, 0, st, x, n, K, out, nullptr, 0);
  return cudaGetLastError();
}
cudaError_t launch_quantize_q8_0_planes(const float* x, int n, int ncols, int K, ActPlanesMut out, cudaStream_t st) {
  const dim3 grid((K / QK32 + 15) / 16, ncols);
  EMELB_LAUNCH(quantize_q8_0_kernel<false>, grid, 128, 0, st, x, n, K, out, nullptr, 0);
  return cudaGetLastError();
}
cudaError_t launch_quantize_q8_k_blocks(const float* x, int n, int K, uint8_t* out, int64_t row_bytes, cudaStream_t st) {
  const dim3 grid((K / QK_K + 3) / 4, n);
  EMELB_LAUNCH(quantize_q8_k_kernel<true>, grid, 128, 0, st, x, n, K, ActPlanesMut{}, out, row_bytes);
  return cudaGetLastError();
}
cudaError_t launch_quantize_q8_0_blocks(const float* x, int n, int K, uint8_t* out, int64_t row_bytes, cudaStream_t st) {
  const dim3 grid((K / QK32 + 15) / 16, n);
  EMELB_LAUNCH(quantize_q8_0_kernel<true>, grid, 128, 0, st, x, n, K, ActPlanesMut{}, out, row_bytes);
  return cudaGetLastError();
}

cudaError_t launch_blocks_to_planes(int type, const uint8_t* blocks, int K, ActPlanesMut out, cudaStream_t st) {
  if (type == T_Q8_K) {
    blocks_to_planes_q8_k_kernel<<<K / QK_K, 64, 0, st>>>(blocks, K / QK_K, out);
  } else if (type == T_Q8_0) {
    blocks_to_planes_q8_0_kernel<<<(K / QK32 + 7) / 8, 128, 0, st>>>(blocks, K / QK32, out);
  } else {
    return cudaErrorInvalidValue;
  }
  return cudaGetLastError();
}

cudaError_t launch_dequantize(int type, const uint8_t* src, int64_t src_row_bytes, float* dst, int64_t dst_row_elems,
                              int K, int M, cudaStream_t st) {
  const dim3 grid((K + 255) / 256, M);
  switch (type) {
    case T_Q4_K: dequantize_kernel<T_Q4_K><<<grid, 256, 0, st>>>(src, src_row_bytes, dst, dst_row_elems, K, M); break;
    case T_Q6_K: dequantize_kernel<T_Q6_K><<<grid, 256, 0, st>>>(src, src_row_bytes, dst, dst_row_elems, K, M); break;
    case T_Q8_0: dequantize_kernel<T_Q8_0><<<grid, 256, 0, st>>>(src, src_row_bytes, dst, dst_row_elems, K, M); break;
    case T_Q4_0: dequantize_kernel<T_Q4_0><<<grid, 256, 0, st>>>(src, src_row_bytes, dst, dst_row_elems, K, M); break;
    default: return cudaErrorInvalidValue;
  }
  return cudaGetLastError();
}

}  // namespace emelb
