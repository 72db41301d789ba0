// Shared device/host definitions for the sm_100a kernels: GGUF block geometry
// (reference: src/emel/kernel/detail.hpp:186-336), the internal activation
// layout, and small PTX helpers.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace emelb {

// dtype codes, src/emel/kernel/events.hpp:78-123
enum : int { T_F32 = 0, T_F16 = 1, T_Q4_0 = 2, T_Q8_0 = 8, T_Q4_K = 12, T_Q6_K = 14, T_Q8_K = 15, T_I32 = 26 };

constexpr int QK_K = 256;
constexpr int QK32 = 32;
constexpr int Q4_K_BYTES = 144;  // u16 d, u16 dmin, u8 scales[12], u8 qs[128]
constexpr int Q6_K_BYTES = 210;  // u8 ql[128], u8 qh[64], i8 scales[16], u16 d
constexpr int Q8_0_BYTES = 34;   // u16 d, i8 qs[32]
constexpr int Q4_0_BYTES = 18;   // u16 d, u8 qs[16]
constexpr int Q8_K_BYTES = 292;  // f32 d, i8 qs[256], i16 bsums[16]
constexpr int MAX_Q8_K_BLOCKS = 128;   // src/emel/kernel/detail.hpp:196
constexpr int MAX_Q8_0_BLOCKS = 1024;  // src/emel/kernel/detail.hpp:197

__host__ __device__ constexpr int block_elems(int t) {
  return (t == T_Q4_K || t == T_Q6_K || t == T_Q8_K) ? 256 : ((t == T_Q8_0 || t == T_Q4_0) ? 32 : 0);
}
__host__ __device__ constexpr int block_bytes(int t) {
  return t == T_Q4_K ? Q4_K_BYTES : t == T_Q6_K ? Q6_K_BYTES : t == T_Q8_0 ? Q8_0_BYTES
       : t == T_Q4_0 ? Q4_0_BYTES : t == T_Q8_K ? Q8_K_BYTES : 0;
}
__host__ __device__ constexpr bool is_k_type(int t) { return t == T_Q4_K || t == T_Q6_K; }

// Quantized activations as the GEMV/GEMM kernels read them.  The reference's
// array-of-blocks layouts (292-byte Q8_K, 34-byte Q8_0) put the int8 payload at
// 4- and 2-byte offsets; on the device the same numbers are kept as separate
// planes so every 16 quants are one aligned 128-bit load.
//   K-quant weights  -> Q8_K planes: qs[n][K] i8, d[n][K/256] f32, bsums[n][K/16] i16
//   32-block weights -> Q8_0 planes: qs[n][K] i8, d[n][K/32]  f32 (= f32 value of
//                       the f16-rounded scale the reference stores)
struct ActPlanes {
  const int8_t* qs;
  const float* d;
  const int16_t* bsums;  // null for Q8_0
  int64_t col_stride_qs;  // = K
  int64_t col_stride_d;   // = K/256 or K/32
  int64_t col_stride_bs;  // = K/16
};

__device__ __forceinline__ float h2f(uint16_t bits) { return __half2float(__ushort_as_half(bits)); }

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
  const uint32_t s = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(s), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory");
}

// Programmatic dependent launch: a kernel launched with the stream-serialization
// attribute may start while its predecessor still runs.  pdl_trigger lets the
// successor start; pdl_wait returns once every predecessor grid has completed
// and its writes are visible.  Both are no-ops for a normal launch.
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

}  // namespace emelb
