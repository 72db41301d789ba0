// Decode attention over the f16 KV cache (one query token per head).
// Replaces run_flash_attn_ext_active_kv_with_workspace_unchecked
// (src/emel/kernel/detail.hpp:5238-5291) and the AVX2 one-chunk route
// (src/emel/kernel/x86_64/actions.hpp:1575-1641).
//
// Two kernels families:
//  * split-KV (default): the KV sequence of each KV head is cut into `splits`
//    ranges, one CTA per (range, kv head, group of <=4 query heads sharing that
//    KV head, so K/V are read once per group).  Inside a CTA: scores for the
//    range (8 lanes per token row, 128-bit loads), exact range maximum,
//    probabilities, then the V accumulation with 128-bit loads; f32 throughout.
//    A small second kernel merges the ranges.  HBM-bound: K and V are each read
//    once.
//  * reference order: scores in the summation order of the reference's scalar
//    route or of its x86 AVX2 route, then the reference's sequential online
//    softmax with an f16 accumulator rounded after every token and libm-exact
//    expf — the same roundings in the same order, for parity runs and for shapes
//    the split kernel does not take.
#include "attention_core.cuh"
#include "common.cuh"
#include "expf_exact.h"
#include "kernels.h"
#include "peer_join.cuh"
#include "quant_device.cuh"

namespace emelb {

namespace {

constexpr int LMAX = 1024;  // tokens per split the shared score buffer holds

template <int D, int NREP>
__global__ void __launch_bounds__(128) flash_split_kernel(const FlashArgs a) {
  pdl_trigger();
  pdl_wait();
  __shared__ __align__(16) float s_p[NREP * LMAX];
  __shared__ float s_red[4 * NREP];
  const int T = a.tokens_dev ? a.tokens_dev[a.kv_heads_per_seq > 0 ? blockIdx.y / a.kv_heads_per_seq : 0] : a.tokens;
  fa::split_unit<D, NREP, LMAX, 8, false>(a, blockIdx.x, blockIdx.y, blockIdx.z, T, threadIdx.x, s_p, s_red, fa::CtaSync{});
}

// merge the ranges (attention_core.cuh).  One CTA of 256 threads = 256 consecutive
// output values (256/D heads), which is also one Q8_K block / eight Q8_0 blocks of the
// vector the output projection consumes, so the CTA can hand the projection its
// quantized planes directly (family 1 / 2; 0 = f32 only).  Warp w < 256/D first turns
// head w's (max, sum) pairs into weights in shared memory; then thread (head, d) walks
// the ranges with independent loads.
using fa::kMergeMaxSplits;

template <int FAMILY>
__global__ void __launch_bounds__(256) flash_merge_kernel(const FlashArgs a, ActPlanesMut planes) {
  pdl_trigger();
  JoinOut jo{};   // a constant of the session: fetched before the wait for the preceding kernel
  if constexpr (FAMILY == 1) {
    if (a.join_out) jo = *a.join_out;
  }
  pdl_wait();
  __shared__ float s_w[4][kMergeMaxSplits];
  __shared__ float s_inv[4];
  __shared__ float s_out[256];
  const int D = a.head_dim, hp = 256 / D;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h0 = blockIdx.x * hp;
  if (warp < hp) fa::merge_head_weights(a, h0 + warp, lane, s_w[warp], &s_inv[warp]);
  __syncthreads();
  const int hl = threadIdx.x / D, d = threadIdx.x - hl * D;
  const float o = fa::merge_output(a, h0 + hl, d, s_w[hl], s_inv[hl]);
  if constexpr (FAMILY == 1) {
    if (a.join_out) {
      // these are this rank's heads of a joined vector: the block goes, quantized, into every rank's planes
      s_out[threadIdx.x] = o;
      __syncthreads();
      if (warp == 0) {
        float v[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = s_out[8 * lane + i];
        uint32_t lo, hi; int bs; float dq;
        q8_k_block_warp(v, lane, lo, hi, bs, dq);
        join_store_q8_k_block(jo, jo.first_block + blockIdx.x, lane, lo, hi, bs, dq);
      }
      join_publish(jo, gridDim.x);
      return;
    }
  }
  if (a.dst_seqs > 1) {
    // several sequences: head h of sequence i is global head i * heads_per_seq + h; dst keeps the sequence index fastest
    const int hps = a.heads / a.dst_seqs, hg = h0 + hl;
    const int seq = hg / hps, hloc = hg - seq * hps;
    a.dst[((size_t)hloc * D + d) * a.dst_seqs + seq] = o;
    if constexpr (FAMILY == 1) {
      // the CTA's 256 values are one Q8_K block of that sequence's column (heads_per_seq * D is a multiple of 256)
      s_out[threadIdx.x] = o;
      __syncthreads();
      if (warp == 0) {
        float v[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = s_out[8 * lane + i];
        uint32_t lo, hi; int bs; float dq;
        q8_k_block_warp(v, lane, lo, hi, bs, dq);
        const int col = (h0 / hps), blk = (h0 - col * hps) * D / QK_K;
        q8_k_store_planes(planes, col, hps * D, blk, lane, lo, hi, bs, dq);
      }
    }
    return;
  } else {
    a.dst[(size_t)h0 * D + threadIdx.x] = o;
  }
  if constexpr (FAMILY != 0) {
    s_out[threadIdx.x] = o;
    __syncthreads();
    const int K = a.heads * D;
    if constexpr (FAMILY == 1) {
      if (warp == 0) {
        float v[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = s_out[8 * lane + i];
        uint32_t lo, hi; int bs; float dq;
        q8_k_block_warp(v, lane, lo, hi, bs, dq);
        q8_k_store_planes(planes, 0, K, blockIdx.x, lane, lo, hi, bs, dq);
      }
    } else {
      if (threadIdx.x < 64) {
        float v[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) v[i] = s_out[4 * threadIdx.x + i];
        uint32_t q; __half dh;
        q8_0_block_oct(v, q, dh);
        const int e0 = blockIdx.x * 256 + 4 * threadIdx.x;
        *reinterpret_cast<uint32_t*>(planes.qs + e0) = q;
        if ((threadIdx.x & 7) == 0) planes.d[e0 / QK32] = __half2float(dh);
      }
    }
  }
}

// any head count: one CTA per head, f32 output only
__global__ void flash_merge_tail_kernel(const FlashArgs a) {
  pdl_trigger();
  pdl_wait();
  const int h = blockIdx.x, D = a.head_dim;
  const float* ml = a.part_ml + (size_t)h * a.splits * 2;
  float M = -INFINITY;
  for (int s = 0; s < a.splits; ++s) M = fmaxf(M, ml[2 * s]);
  float den = 0.0f;
  for (int s = 0; s < a.splits; ++s) den += (ml[2 * s] == -INFINITY ? 0.0f : expf(ml[2 * s] - M)) * ml[2 * s + 1];
  const float inv = den == 0.0f ? 0.0f : 1.0f / den;
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float o = 0.0f;
    for (int s = 0; s < a.splits; ++s) {
      const float w = ml[2 * s] == -INFINITY ? 0.0f : expf(ml[2 * s] - M);
      o = fmaf(w, a.part_acc[((size_t)h * a.splits + s) * D + d], o);
    }
    a.dst[(size_t)h * D + d] = o * inv;
  }
}

// ---------------------------------------------------------------- reference order
// scores[h][t] in one of the reference's two summation orders; one warp per
// (token, head):
//  order 1 (scalar route): (float)(sum_i (double)q16[i] * (double)k[t][i]) * scale
//    (dot_product_f16_f16_scores, src/emel/kernel/detail.hpp:2203-2208), f64
//    partial sums combined across lanes;
//  order 2 (x86 AVX2 route): four 8-lane f32 accumulators advanced by fused
//    multiply-adds 32 elements at a time, folded (0+1)+(2+3) in f32, the 8 lanes
//    then summed in f64 in lane order, the tail (< 32 elements) added as f64
//    products (dot_product_f16_f16_scores_avx2_fma,
//    src/emel/kernel/x86_64/actions.hpp:1388-1446).  Warp lane L = 8j + l plays
//    lane l of accumulator j, so every rounding happens where the AVX2 code has it.
__global__ void __launch_bounds__(128) flash_ref_scores_kernel(const FlashArgs a, float* scores, int t_stride, int order) {
  pdl_trigger();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int T = a.tokens_dev ? *a.tokens_dev : a.tokens;
  const int h = blockIdx.y;
  const int kh = h / (a.heads / a.kv_heads);
  const int D = a.head_dim;
  const float* qh = a.q + (size_t)h * D;
  for (int t = blockIdx.x * 4 + (threadIdx.x >> 5); t < T; t += gridDim.x * 4) {
    const __half* kr = reinterpret_cast<const __half*>(reinterpret_cast<const char*>(a.k) + (size_t)t * a.k_nb1 + (size_t)kh * a.k_nb2);
    double s = 0.0;
    if (order == 2) {
      const int vec = D & ~31;
      float f = 0.0f;
      for (int i = lane; i < vec; i += 32) f = __fmaf_rn(__half2float(__float2half_rn(qh[i])), __half2float(kr[i]), f);
      f = __fadd_rn(f, __shfl_xor_sync(0xffffffffu, f, 8));    // sum0+sum1 | sum2+sum3
      f = __fadd_rn(f, __shfl_xor_sync(0xffffffffu, f, 16));   // (sum0+sum1)+(sum2+sum3)
      for (int l = 0; l < 8; ++l) s += (double)__shfl_sync(0xffffffffu, f, l);
      for (int i = vec; i < D; ++i) s += (double)__half2float(__float2half_rn(qh[i])) * (double)__half2float(kr[i]);
    } else {
      for (int i = lane; i < D; i += 32) s += (double)__half2float(__float2half_rn(qh[i])) * (double)__half2float(kr[i]);
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    }
    if (lane == 0) scores[(size_t)h * t_stride + t] = __fmul_rn((float)s, a.scale);
  }
}

__device__ __forceinline__ float round16(float v) { return __half2float(__float2half_rn(v)); }

// One CTA per head; thread d owns accumulator dims d, d+blockDim, ...; every
// thread replays the scalar recurrences (max, scales, sum) so no barrier sits
// inside the token loop.  Mirrors detail.hpp:5261-5290 with
// scale_f16_buffer_scalar (:4312-4320) and axpy_f16_buffer_scalar (:4322-4332).
template <int DPT>
__global__ void flash_ref_sequential_kernel(const FlashArgs a, const float* scores, int t_stride) {
  pdl_trigger();
  pdl_wait();
  __shared__ float s_sc[256];
  const int T = a.tokens_dev ? *a.tokens_dev : a.tokens;
  const int h = blockIdx.x, D = a.head_dim;
  const int kh = h / (a.heads / a.kv_heads);
  float acc[DPT];
#pragma unroll
  for (int i = 0; i < DPT; ++i) acc[i] = 0.0f;
  float sum = 0.0f, mx = -INFINITY;
  const char* vbase = reinterpret_cast<const char*>(a.v) + (size_t)kh * a.v_nb2;
  for (int tb = 0; tb < T; tb += 256) {
    __syncthreads();
    for (int i = threadIdx.x; i < 256 && tb + i < T; i += blockDim.x) s_sc[i] = scores[(size_t)h * t_stride + tb + i];
    __syncthreads();
    const int tn = min(256, T - tb);
    for (int tt = 0; tt < tn; ++tt) {
      const float score = s_sc[tt];
      const float old = mx;
      float ms = 1.0f, vsc = 1.0f;
      const bool bump = score > mx;
      if (bump) { mx = score; ms = expf_exact(old - mx); } else { vsc = expf_exact(score - mx); }
      const float rs = round16(ms), ra = round16(vsc);
      const __half* vr = reinterpret_cast<const __half*>(vbase + (size_t)(tb + tt) * a.v_nb1);
#pragma unroll
      for (int i = 0; i < DPT; ++i) {
        const int d = threadIdx.x + i * blockDim.x;
        if (d < D) {
          float x = acc[i];
          if (bump) x = round16(__fmul_rn(x, rs));
          acc[i] = round16(__fadd_rn(x, __fmul_rn(__half2float(vr[d]), ra)));
        }
      }
      sum = __fadd_rn(__fmul_rn(sum, ms), vsc);
    }
  }
  const float inv = sum == 0.0f ? 0.0f : __fdiv_rn(1.0f, sum);
#pragma unroll
  for (int i = 0; i < DPT; ++i) {
    const int d = threadIdx.x + i * blockDim.x;
    if (d < D) a.dst[(size_t)h * D + d] = sum == 0.0f ? 0.0f : __fmul_rn(acc[i], inv);
  }
}

template <int D>
cudaError_t launch_split(const FlashArgs& a, int n_rep, cudaStream_t st) {
  if (n_rep % 4 == 0) {
    EMELB_LAUNCH((flash_split_kernel<D, 4>), dim3(a.splits, a.kv_heads, n_rep / 4), 128, 0, st, a);
  } else if (n_rep % 2 == 0) {
    EMELB_LAUNCH((flash_split_kernel<D, 2>), dim3(a.splits, a.kv_heads, n_rep / 2), 128, 0, st, a);
  } else {
    EMELB_LAUNCH((flash_split_kernel<D, 1>), dim3(a.splits, a.kv_heads, n_rep), 128, 0, st, a);
  }
  return cudaGetLastError();
}

}  // namespace

int flash_pick_splits(int tokens, int kv_heads, int sm_count, int max_splits) {
  int need = (tokens + LMAX - 1) / LMAX;          // score buffer bound
  int want = (2 * sm_count + kv_heads - 1) / kv_heads;  // ~2 CTAs per SM (3 and 4 measured slower in the decode loop)
  const int by_len = tokens / 32 > 0 ? tokens / 32 : 1; // at least 32 tokens per range
  if (want > by_len) want = by_len;
  if (want < need) want = need;
  if (want > max_splits) want = max_splits;
  return want < 1 ? 1 : want;
}

bool flash_split_supported(const FlashArgs& a) {
  const bool d_ok = a.head_dim == 64 || a.head_dim == 128;
  const bool al = (reinterpret_cast<uintptr_t>(a.k) % 16 == 0) && (reinterpret_cast<uintptr_t>(a.v) % 16 == 0) &&
                  (reinterpret_cast<uintptr_t>(a.q) % 16 == 0) &&
                  a.k_nb1 % 16 == 0 && a.k_nb2 % 16 == 0 && a.v_nb1 % 16 == 0 && a.v_nb2 % 16 == 0;
  return d_ok && al && (int64_t)a.splits * LMAX >= a.tokens;
}

bool flash_merge_can_quantize(const FlashArgs& a) { return (a.heads * a.head_dim) % 256 == 0; }

cudaError_t launch_flash_decode(const FlashArgs& a, int sm_count, cudaStream_t st, int* launches, int out_family,
                                ActPlanesMut out_planes) {
  (void)sm_count;
  if (a.join_out && (a.heads * a.head_dim) % 256 != 0) return cudaErrorInvalidValue;
  const int n_rep = a.heads / a.kv_heads;
  cudaError_t e = a.head_dim == 64 ? launch_split<64>(a, n_rep, st) : launch_split<128>(a, n_rep, st);
  if (e != cudaSuccess) return e;
  const int total = a.heads * a.head_dim;
  if (total % 256 == 0) {
    if (a.join_out) out_family = 1;
    if (out_family == 1) EMELB_LAUNCH(flash_merge_kernel<1>, total / 256, 256, 0, st, a, out_planes);
    else if (out_family == 2) EMELB_LAUNCH(flash_merge_kernel<2>, total / 256, 256, 0, st, a, out_planes);
    else EMELB_LAUNCH(flash_merge_kernel<0>, total / 256, 256, 0, st, a, out_planes);
  } else {
    EMELB_LAUNCH(flash_merge_tail_kernel, a.heads, 128, 0, st, a);   // head counts that do not fill 256-value groups
  }
  *launches += 2;
  return cudaGetLastError();
}

cudaError_t launch_flash_reference_order(const FlashArgs& a, float* score_ws, int t_stride, int order, cudaStream_t st,
                                         int* launches) {
  int gx = (a.tokens + 3) / 4;
  if (gx > 1024) gx = 1024;
  EMELB_LAUNCH(flash_ref_scores_kernel, dim3(gx, a.heads), 128, 0, st, a, score_ws, t_stride, order);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  const int D = a.head_dim;
  if (D <= 256) EMELB_LAUNCH(flash_ref_sequential_kernel<1>, a.heads, D < 32 ? 32 : ((D + 31) / 32) * 32, 0, st, a, score_ws, t_stride);
  else if (D <= 1024) EMELB_LAUNCH(flash_ref_sequential_kernel<4>, a.heads, 256, 0, st, a, score_ws, t_stride);
  else EMELB_LAUNCH(flash_ref_sequential_kernel<16>, a.heads, 256, 0, st, a, score_ws, t_stride);
  *launches += 2;
  return cudaGetLastError();
}

}  // namespace emelb
