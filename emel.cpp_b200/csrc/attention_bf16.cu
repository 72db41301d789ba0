// kernel::attention's head-range event on the device: one query token against a bf16 KV ring buffer
// (src/emel/kernel/attention/actions.hpp:15-96), in the arithmetic of the reference's scalar route:
//   q -> bf16 (ggml rounding, src/emel/kernel/detail.hpp:3944-3952);
//   score[p] = (float)(sum_i (double)(k_i * q_i)) * scale, products in f32, sum in element order
//              (vec_dot_bf16_ggml's scalar loop, :3990-3993);
//   softmax over all `capacity` rows (soft_max_row_ggml's scalar loop, :4122-4157): max, expf, an f64 sum in row
//              order, weights = e * (float)(1 / sum); rows outside the valid range hold -inf -> weight 0;
//   weights -> bf16; out[d] = (float)(sum_p (double)(v[p][d] * w[p])) over the valid positions in logical order.
// Every sum whose order the reference fixes is kept sequential here: one thread per position walks the head's
// elements, one thread adds the row's exponentials, one thread per output element walks the positions.  It is a
// parity kernel for an operator outside the decode loop, not a throughput kernel.
// Compiled with -fmad=false; expf is the table-and-polynomial expf whose bits equal glibc's (expf_exact.h).
#include "common.cuh"
#include "expf_exact.h"
#include "kernels.h"

namespace emelb {

namespace {

__device__ __forceinline__ float bf16_bits_to_f32(uint16_t b) { return __uint_as_float((uint32_t)b << 16); }
// round to nearest even, NaNs quieted (src/emel/kernel/detail.hpp:3944-3952)
__device__ __forceinline__ uint16_t f32_to_bf16_bits(float v) {
  const uint32_t u = __float_as_uint(v);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 64u);
  return (uint16_t)((u + (0x7fffu + ((u >> 16) & 1u))) >> 16);
}

__global__ void __launch_bounds__(256) head_range_attention_kernel(const HeadRangeArgs a) {
  extern __shared__ __align__(16) float smem_hr[];
  float* s_q = smem_hr;                         // head_dim: the query rounded to bf16
  float* s_w = smem_hr + a.head_dim;            // capacity: scores, then exponentials, then bf16-rounded weights
  __shared__ float s_red[256];
  __shared__ float s_inv;
  const int head = a.head_begin + blockIdx.x, head_offset = head * a.head_dim;
  const int tid = threadIdx.x, nthreads = blockDim.x;
  for (int d = tid; d < a.head_dim; d += nthreads) s_q[d] = bf16_bits_to_f32(f32_to_bf16_bits(a.query[head_offset + d]));
  for (int p = tid; p < a.capacity; p += nthreads) s_w[p] = -INFINITY;
  __syncthreads();
  // scores of the valid positions
  for (int pos = tid; pos < a.valid; pos += nthreads) {
    const int64_t un = (int64_t)a.physical_begin + pos;
    const int physical = (int)(un - (un >= a.capacity ? a.capacity : 0));
    const uint16_t* k = a.key + a.layer_offset + (size_t)physical * a.hidden_dim + head_offset;
    double sum = 0.0;
    for (int i = 0; i < a.head_dim; ++i) sum += (double)__fmul_rn(bf16_bits_to_f32(k[i]), s_q[i]);
    s_w[physical] = __fmul_rn((float)sum, a.scale);
  }
  __syncthreads();
  // max over every row (the order of a max does not matter)
  float mx = -INFINITY;
  for (int p = tid; p < a.capacity; p += nthreads) mx = fmaxf(mx, s_w[p]);
  s_red[tid] = mx;
  __syncthreads();
  for (int o = 128; o > 0; o >>= 1) {
    if (tid < o && tid + o < nthreads) s_red[tid] = fmaxf(s_red[tid], s_red[tid + o]);
    __syncthreads();
  }
  mx = s_red[0];
  for (int p = tid; p < a.capacity; p += nthreads) {
    const float x = __fsub_rn(s_w[p], mx);
    s_w[p] = x == -INFINITY ? 0.0f : expf_exact(x);
  }
  __syncthreads();
  if (tid == 0) {
    double sum = 0.0;
    for (int p = 0; p < a.capacity; ++p) sum += (double)s_w[p];   // row order, as the reference adds them
    s_inv = (float)(1.0 / sum);
  }
  __syncthreads();
  const float inv = s_inv;
  for (int p = tid; p < a.capacity; p += nthreads) s_w[p] = bf16_bits_to_f32(f32_to_bf16_bits(__fmul_rn(s_w[p], inv)));
  __syncthreads();
  // weighted sum of the value rows, valid positions in logical order
  for (int d = tid; d < a.head_dim; d += nthreads) {
    double acc = 0.0;
    for (int pos = 0; pos < a.valid; ++pos) {
      const int64_t un = (int64_t)a.physical_begin + pos;
      const int physical = (int)(un - (un >= a.capacity ? a.capacity : 0));
      const float v = bf16_bits_to_f32(a.value[a.layer_offset + (size_t)physical * a.hidden_dim + head_offset + d]);
      acc += (double)__fmul_rn(v, s_w[physical]);
    }
    a.output[(size_t)blockIdx.x * a.head_dim + d] = (float)acc;
  }
}

}  // namespace

cudaError_t launch_head_range_attention(const HeadRangeArgs& a, cudaStream_t st) {
  const size_t smem = sizeof(float) * ((size_t)a.head_dim + (size_t)a.capacity);
  static thread_local unsigned configured = 0;  // one bit per device (one context, one lane per host thread)
  int dev = 0;
  cudaGetDevice(&dev);
  if (!(configured & (1u << (dev & 31)))) {
    const cudaError_t e = cudaFuncSetAttribute(head_range_attention_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 4 * 2 * 8192);
    if (e != cudaSuccess) return e;
    configured |= 1u << (dev & 31);
  }
  head_range_attention_kernel<<<a.head_end - a.head_begin, 256, smem, st>>>(a);
  return cudaGetLastError();
}

}  // namespace emelb
