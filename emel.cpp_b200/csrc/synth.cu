// Synthetic model data generated on the device: N(0, sigma) f32 values from a
// counter-based generator, and this project's own encoders from f32 to the four
// GGUF block formats (the reference has no K-quant encoder; any encoder that
// emits valid blocks serves, since every consumer reads the same bytes).  Used
// to fill benchmark-sized weight matrices (tens of GB) without a host pass.
#include "common.cuh"
#include "kernels.h"

namespace emelb {

namespace {

__device__ __forceinline__ uint32_t mix32(uint64_t z) {
  z += 0x9e3779b97f4a7c15ull;
  z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
  z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
  return (uint32_t)((z ^ (z >> 31)) >> 16);
}

// standard normal by Box-Muller over two hashed uniforms of the element index
__device__ __forceinline__ float normal_at(uint64_t seed, uint64_t idx) {
  const uint32_t a = mix32(seed * 0x100000001b3ull + 2 * idx);
  const uint32_t b = mix32(seed * 0x100000001b3ull + 2 * idx + 1);
  const float u1 = ((float)a + 1.0f) * (1.0f / 4294967296.0f);
  const float u2 = (float)b * (1.0f / 4294967296.0f);
  return sqrtf(-2.0f * logf(u1)) * cospif(2.0f * u2);
}

__global__ void fill_normal_kernel(float* out, uint64_t n, uint64_t seed, float sigma, uint64_t offset) {
  for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x)
    out[i] = sigma * normal_at(seed, offset + i);
}

__device__ __forceinline__ uint16_t f2h_bits(float f) { return __half_as_ushort(__float2half_rn(f)); }

// one thread per 256-element super-block (encoders are setup code, not a hot path)
__global__ void encode_k_kernel(int type, uint8_t* out, uint64_t nblocks, uint64_t seed, float sigma, uint64_t elem_offset) {
  const uint64_t b = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= nblocks) return;
  float x[256];
  for (int i = 0; i < 256; ++i) x[i] = sigma * normal_at(seed, elem_offset + b * 256 + i);
  uint8_t blk[Q6_K_BYTES];
  uint8_t* const y = blk;
  if (type == T_Q4_K) {
    float sc[8], mn[8], max_sc = 0.0f, max_mn = 0.0f;
    for (int j = 0; j < 8; ++j) {
      float lo = x[32 * j], hi = x[32 * j];
      for (int l = 1; l < 32; ++l) { lo = fminf(lo, x[32 * j + l]); hi = fmaxf(hi, x[32 * j + l]); }
      lo = fminf(lo, 0.0f);
      sc[j] = (hi - lo) / 15.0f;
      mn[j] = -lo;
      max_sc = fmaxf(max_sc, sc[j]);
      max_mn = fmaxf(max_mn, mn[j]);
    }
    const uint16_t dh = f2h_bits(max_sc / 63.0f), mh = f2h_bits(max_mn / 63.0f);
    const float dq = h2f(dh), dmq = h2f(mh);
    y[0] = dh & 0xff; y[1] = dh >> 8; y[2] = mh & 0xff; y[3] = mh >> 8;
    int ls[8], lm[8];
    for (int j = 0; j < 8; ++j) {
      ls[j] = dq > 0.0f ? min(63, max(0, __float2int_rn(sc[j] / dq))) : 0;
      lm[j] = dmq > 0.0f ? min(63, max(0, __float2int_rn(mn[j] / dmq))) : 0;
    }
    uint8_t s[12];
    for (int i = 0; i < 12; ++i) s[i] = 0;
    for (int j = 0; j < 8; ++j) {
      if (j < 4) { s[j] = (uint8_t)ls[j]; s[j + 4] = (uint8_t)lm[j]; }
      else {
        s[j + 4] = (uint8_t)((ls[j] & 0x0f) | ((lm[j] & 0x0f) << 4));
        s[j - 4] |= (uint8_t)((ls[j] >> 4) << 6);
        s[j] |= (uint8_t)((lm[j] >> 4) << 6);
      }
    }
    for (int i = 0; i < 12; ++i) y[4 + i] = s[i];
    for (int g = 0; g < 4; ++g) {
      const float d0 = dq * ls[2 * g], m0 = dmq * lm[2 * g], d1 = dq * ls[2 * g + 1], m1 = dmq * lm[2 * g + 1];
      for (int l = 0; l < 32; ++l) {
        const int a = d0 > 0.0f ? min(15, max(0, __float2int_rn((x[64 * g + l] + m0) / d0))) : 0;
        const int c = d1 > 0.0f ? min(15, max(0, __float2int_rn((x[64 * g + 32 + l] + m1) / d1))) : 0;
        y[16 + 32 * g + l] = (uint8_t)(a | (c << 4));
      }
    }
  } else {  // T_Q6_K
    float gs[16], mx = 0.0f;
    for (int g = 0; g < 16; ++g) {
      float am = 0.0f;
      for (int l = 0; l < 16; ++l) am = fmaxf(am, fabsf(x[16 * g + l]));
      gs[g] = am / 31.0f;
      mx = fmaxf(mx, gs[g]);
    }
    const uint16_t dh = f2h_bits(mx / 127.0f);
    const float dq = h2f(dh);
    y[208] = dh & 0xff; y[209] = dh >> 8;
    uint8_t q[256];
    for (int g = 0; g < 16; ++g) {
      int s = dq > 0.0f ? min(127, __float2int_rn(gs[g] / dq)) : 0;
      if (s < 1 && gs[g] > 0.0f) s = 1;
      y[192 + g] = (uint8_t)(int8_t)s;
      const float step = dq * s;
      for (int l = 0; l < 16; ++l) {
        const int v = step > 0.0f ? min(31, max(-32, __float2int_rn(x[16 * g + l] / step))) : 0;
        q[16 * g + l] = (uint8_t)(v + 32);
      }
    }
    for (int n = 0; n < 2; ++n)
      for (int l = 0; l < 32; ++l) {
        const uint8_t q1 = q[128 * n + l], q2 = q[128 * n + l + 32], q3 = q[128 * n + l + 64], q4 = q[128 * n + l + 96];
        y[64 * n + l] = (uint8_t)((q1 & 0x0f) | ((q3 & 0x0f) << 4));
        y[64 * n + l + 32] = (uint8_t)((q2 & 0x0f) | ((q4 & 0x0f) << 4));
        y[128 + 32 * n + l] = (uint8_t)((q1 >> 4) | ((q2 >> 4) << 2) | ((q3 >> 4) << 4) | ((q4 >> 4) << 6));
      }
  }
  // blocks are 2-byte aligned in the destination: copy as 16-bit words
  const int bytes = type == T_Q4_K ? Q4_K_BYTES : Q6_K_BYTES;
  uint16_t* dst = reinterpret_cast<uint16_t*>(out + b * bytes);
  for (int i = 0; i < bytes / 2; ++i) dst[i] = (uint16_t)blk[2 * i] | ((uint16_t)blk[2 * i + 1] << 8);
}

// one thread per 32-element block
__global__ void encode_32_kernel(int type, uint8_t* out, uint64_t nblocks, uint64_t seed, float sigma, uint64_t elem_offset) {
  const uint64_t b = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= nblocks) return;
  float x[32];
  float amax = 0.0f, mx = 0.0f;
  for (int i = 0; i < 32; ++i) {
    x[i] = sigma * normal_at(seed, elem_offset + b * 32 + i);
    if (fabsf(x[i]) > amax) { amax = fabsf(x[i]); mx = x[i]; }
  }
  uint8_t blk[Q8_0_BYTES];
  uint8_t* const y = blk;
  if (type == T_Q8_0) {
    const float d = amax / 127.0f, id = d != 0.0f ? 1.0f / d : 0.0f;
    const uint16_t dh = f2h_bits(d);
    y[0] = dh & 0xff; y[1] = dh >> 8;
    for (int i = 0; i < 32; ++i) y[2 + i] = (uint8_t)(int8_t)max(-127, min(127, (int)roundf(x[i] * id)));
  } else {
    const float d = mx / -8.0f, id = d != 0.0f ? 1.0f / d : 0.0f;
    const uint16_t dh = f2h_bits(d);
    y[0] = dh & 0xff; y[1] = dh >> 8;
    for (int j = 0; j < 16; ++j) {
      const int a = max(0, min(15, (int)(x[j] * id + 8.5f)));
      const int c = max(0, min(15, (int)(x[j + 16] * id + 8.5f)));
      y[2 + j] = (uint8_t)(a | (c << 4));
    }
  }
  const int bytes = type == T_Q8_0 ? Q8_0_BYTES : Q4_0_BYTES;
  uint16_t* dst = reinterpret_cast<uint16_t*>(out + b * bytes);
  for (int i = 0; i < bytes / 2; ++i) dst[i] = (uint16_t)blk[2 * i] | ((uint16_t)blk[2 * i + 1] << 8);
}

}  // namespace

cudaError_t launch_fill_normal(float* out, uint64_t n, uint64_t seed, float sigma, uint64_t offset, cudaStream_t st) {
  uint64_t blocks = (n + 255) / 256;
  if (blocks > 65535) blocks = 65535;
  fill_normal_kernel<<<(unsigned)blocks, 256, 0, st>>>(out, n, seed, sigma, offset);
  return cudaGetLastError();
}

cudaError_t launch_encode_normal(int type, uint8_t* out, uint64_t elems, uint64_t seed, float sigma, uint64_t offset,
                                 cudaStream_t st) {
  const uint64_t nblocks = elems / block_elems(type);
  if (nblocks == 0) return cudaErrorInvalidValue;
  const uint64_t grid = (nblocks + 63) / 64;
  if (grid > 0x7fffffffull) return cudaErrorInvalidValue;
  if (is_k_type(type)) encode_k_kernel<<<(unsigned)grid, 64, 0, st>>>(type, out, nblocks, seed, sigma, offset);
  else if (type == T_Q8_0 || type == T_Q4_0) encode_32_kernel<<<(unsigned)grid, 64, 0, st>>>(type, out, nblocks, seed, sigma, offset);
  else return cudaErrorInvalidValue;
  return cudaGetLastError();
}

}  // namespace emelb
