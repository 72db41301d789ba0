/*
 * TEST INFRASTRUCTURE ONLY — a CPU restatement, in plain C, of the reference's
 * quantized matrix-product path.  Nothing in the product path may include,
 * link or call this file; it exists to check the CUDA kernels (tests/, the
 * smoke check, the bench's cpu_baseline leg).
 *
 * Every function cites the reference lines it restates (paths relative to the
 * reference checkout).  Build: gcc -O2 -std=c11 -ffp-contract=off (see
 * oracle/Makefile) — contraction off so float expressions round exactly as
 * written, the same build definition as oracle/_ref.
 *
 * Parity status: pinned.  tests/test_oracle.py checks this file against the
 * reference's own known-answer tests and against oracle/_ref (the reference's
 * headers compiled in place) on seeded inputs; tests/golden holds vectors
 * generated from oracle/_ref.  Exception: the Q4_K/Q6_K *weight* encoders at
 * the bottom are this project's own design (the reference only consumes those
 * blocks; its encoder lives in ggml, which is not vendored) — "parity
 * unpinned" for those two encoders only; both sides of every parity check
 * consume the same bytes.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define QK_K 256
#define QK8_0 32
#define QK4_0 32
#define MAX_Q8_K_BLOCKS 128  /* src/emel/kernel/detail.hpp:196 */
#define MAX_Q8_0_BLOCKS 1024 /* src/emel/kernel/detail.hpp:197 */

enum { T_F32 = 0, T_F16 = 1, T_Q4_0 = 2, T_Q8_0 = 8, T_Q4_K = 12, T_Q6_K = 14, T_Q8_K = 15 };

#pragma pack(push, 1)
/* src/emel/kernel/detail.hpp:202-205 */
typedef struct { uint16_t d; uint8_t qs[16]; } blk_q4_0;
/* src/emel/kernel/detail.hpp:226-229 */
typedef struct { uint16_t d; int8_t qs[32]; } blk_q8_0;
/* src/emel/kernel/detail.hpp:250-255 */
typedef struct { uint16_t d; uint16_t dmin; uint8_t scales[12]; uint8_t qs[128]; } blk_q4_k;
/* src/emel/kernel/detail.hpp:265-270 */
typedef struct { uint8_t ql[128]; uint8_t qh[64]; int8_t scales[16]; uint16_t d; } blk_q6_k;
/* src/emel/kernel/detail.hpp:298-302 */
typedef struct { float d; int8_t qs[256]; int16_t bsums[16]; } blk_q8_k;
#pragma pack(pop)

_Static_assert(sizeof(blk_q4_0) == 18, "q4_0");
_Static_assert(sizeof(blk_q8_0) == 34, "q8_0");
_Static_assert(sizeof(blk_q4_k) == 144, "q4_k");
_Static_assert(sizeof(blk_q6_k) == 210, "q6_k");
_Static_assert(sizeof(blk_q8_k) == 292, "q8_k");

/* mirrors emelb_view / emelb_op (include/emelb.h), kept local so this file
 * stands alone */
typedef struct { const void* data; uint8_t type; uint64_t ne[4]; uint64_t nb[4]; } o_view;
typedef struct { o_view src0, src1, src2, dst; uint8_t op_params[64]; uint32_t op_params_size; int32_t* index_out; } o_op;

static float bits_f32(uint32_t b) { float f; memcpy(&f, &b, 4); return f; }
static uint32_t f32_bits(float f) { uint32_t b; memcpy(&b, &f, 4); return b; }

/* src/emel/kernel/detail.hpp:350-370 */
float orc_fp16_to_fp32(uint16_t h) {
  const uint32_t w = (uint32_t)h << 16;
  const uint32_t sign = w & 0x80000000u;
  const uint32_t two_w = w + w;
  const float normalized = bits_f32((two_w >> 4) + (0xE0u << 23)) * 0x1.0p-112f;
  const float denormalized = bits_f32((two_w >> 17) | (126u << 23)) - 0.5f;
  const uint32_t r = sign | (two_w < (1u << 27) ? f32_bits(denormalized) : f32_bits(normalized));
  return bits_f32(r);
}

/* src/emel/kernel/detail.hpp:372-392 */
uint16_t orc_fp32_to_fp16(float f) {
  float base = (fabsf(f) * 0x1.0p+112f) * 0x1.0p-110f;
  const uint32_t w = f32_bits(f);
  const uint32_t shl1_w = w + w;
  const uint32_t sign = w & 0x80000000u;
  uint32_t bias = shl1_w & 0xFF000000u;
  if (bias < 0x71000000u) bias = 0x71000000u;
  base = bits_f32((bias >> 1) + 0x07800000u) + base;
  const uint32_t bits = f32_bits(base);
  const uint32_t exp_bits = (bits >> 13) & 0x00007C00u;
  const uint32_t mantissa_bits = bits & 0x00000FFFu;
  const uint32_t nonsign = exp_bits + mantissa_bits;
  return (uint16_t)((sign >> 16) | (shl1_w > 0xFF000000u ? 0x7E00u : nonsign));
}

/* src/emel/kernel/detail.hpp:692-697 */
static int nearest_int(float v) {
  float biased = v + 12582912.0f;
  int bits; memcpy(&bits, &biased, 4);
  return (bits & 0x007fffff) - 0x00400000;
}

/* src/emel/kernel/detail.hpp:826-867 */
void orc_quantize_q8_k(const float* x, uint64_t stride, void* out, int64_t k) {
  blk_q8_k* y = (blk_q8_k*)out;
  const int64_t nb = k / QK_K;
  for (int64_t i = 0; i < nb; ++i) {
    const float* blk = x + i * QK_K * (int64_t)stride;
    float max = 0.0f, amax = 0.0f;
    for (int j = 0; j < QK_K; ++j) {
      const float v = blk[(uint64_t)j * stride];
      const float a = fabsf(v);
      if (a > amax) { amax = a; max = v; }
    }
    if (amax == 0.0f) { memset(&y[i], 0, sizeof(blk_q8_k)); continue; }
    const float iscale = -127.0f / max;
    for (int j = 0; j < QK_K; ++j) {
      const int q = nearest_int(iscale * blk[(uint64_t)j * stride]);
      y[i].qs[j] = (int8_t)(q < 127 ? q : 127);
    }
    for (int j = 0; j < QK_K / 16; ++j) {
      int s = 0;
      for (int l = 0; l < 16; ++l) s += y[i].qs[j * 16 + l];
      y[i].bsums[j] = (int16_t)s;
    }
    y[i].d = 1.0f / iscale;
  }
}

/* src/emel/kernel/detail.hpp:804-824 (std::round = half away from zero) */
void orc_quantize_q8_0(const float* x, uint64_t stride, void* out, int64_t k) {
  blk_q8_0* y = (blk_q8_0*)out;
  const int64_t nb = k / QK8_0;
  for (int64_t i = 0; i < nb; ++i) {
    const float* blk = x + i * QK8_0 * (int64_t)stride;
    float amax = 0.0f;
    for (int j = 0; j < QK8_0; ++j) {
      const float a = fabsf(blk[(uint64_t)j * stride]);
      amax = amax < a ? a : amax; /* std::max(amax, a) */
    }
    const float d = amax / 127.0f;
    const float id = d != 0.0f ? 1.0f / d : 0.0f;
    y[i].d = orc_fp32_to_fp16(d);
    for (int j = 0; j < QK8_0; ++j) {
      int q = (int)roundf(blk[(uint64_t)j * stride] * id);
      if (q < -127) q = -127;
      if (q > 127) q = 127;
      y[i].qs[j] = (int8_t)q;
    }
  }
}

/* src/emel/kernel/detail.hpp:699-729 (the one 4-bit weight encoder the
 * reference owns) */
void orc_quantize_q4_0(const float* x, void* out, int64_t k) {
  blk_q4_0* y = (blk_q4_0*)out;
  const int64_t nb = k / QK4_0;
  for (int64_t i = 0; i < nb; ++i) {
    const float* blk = x + i * QK4_0;
    float amax = 0.0f, max = 0.0f;
    for (int j = 0; j < QK4_0; ++j) {
      const float a = fabsf(blk[j]);
      if (a > amax) { amax = a; max = blk[j]; }
    }
    const float d = max / -8.0f;
    const float id = d != 0.0f ? 1.0f / d : 0.0f;
    y[i].d = orc_fp32_to_fp16(d);
    for (int j = 0; j < QK4_0 / 2; ++j) {
      const float x0 = blk[j] * id;
      const float x1 = blk[j + QK4_0 / 2] * id;
      int a = (int)(x0 + 8.5f), b = (int)(x1 + 8.5f);
      a = a < 0 ? 0 : (a > 15 ? 15 : a);
      b = b < 0 ? 0 : (b > 15 ? 15 : b);
      y[i].qs[j] = (uint8_t)((a & 0x0f) | ((b & 0x0f) << 4));
    }
  }
}

/* src/emel/kernel/detail.hpp:475-485 */
static void scale_min_k4(int j, const uint8_t* q, uint8_t* d, uint8_t* m) {
  if (j < 4) { *d = q[j] & 63; *m = q[j + 4] & 63; return; }
  *d = (uint8_t)((q[j + 4] & 0x0f) | ((q[j - 4] >> 6) << 4));
  *m = (uint8_t)((q[j + 4] >> 4) | ((q[j] >> 6) << 4));
}

/* src/emel/kernel/detail.hpp:487-502, 523-552, 592-629, 679-690 */
int orc_dequantize_row(int type, const void* src, float* y, int64_t k) {
  if (type == T_Q4_0) {
    const blk_q4_0* x = (const blk_q4_0*)src;
    for (int64_t i = 0; i < k / QK4_0; ++i) {
      const float d = orc_fp16_to_fp32(x[i].d);
      for (int j = 0; j < 16; ++j) {
        y[i * 32 + j] = (float)((int)(x[i].qs[j] & 0x0f) - 8) * d;
        y[i * 32 + j + 16] = (float)((int)(x[i].qs[j] >> 4) - 8) * d;
      }
    }
    return 1;
  }
  if (type == T_Q8_0) {
    const blk_q8_0* x = (const blk_q8_0*)src;
    for (int64_t i = 0; i < k / QK8_0; ++i) {
      const float d = orc_fp16_to_fp32(x[i].d);
      for (int j = 0; j < 32; ++j) y[i * 32 + j] = d * (float)x[i].qs[j];
    }
    return 1;
  }
  if (type == T_Q4_K) {
    const blk_q4_k* x = (const blk_q4_k*)src;
    for (int64_t i = 0; i < k / QK_K; ++i) {
      const uint8_t* q = x[i].qs;
      const float d = orc_fp16_to_fp32(x[i].d);
      const float mn = orc_fp16_to_fp32(x[i].dmin);
      int is = 0;
      for (int j = 0; j < QK_K; j += 64) {
        uint8_t sc, m;
        scale_min_k4(is + 0, x[i].scales, &sc, &m);
        const float d0 = d * (float)sc, m0 = mn * (float)m;
        scale_min_k4(is + 1, x[i].scales, &sc, &m);
        const float d1 = d * (float)sc, m1 = mn * (float)m;
        for (int l = 0; l < 32; ++l) *y++ = d0 * (float)(q[l] & 0x0f) - m0;
        for (int l = 0; l < 32; ++l) *y++ = d1 * (float)(q[l] >> 4) - m1;
        q += 32; is += 2;
      }
    }
    return 1;
  }
  if (type == T_Q6_K) {
    const blk_q6_k* x = (const blk_q6_k*)src;
    for (int64_t i = 0; i < k / QK_K; ++i) {
      const float d = orc_fp16_to_fp32(x[i].d);
      const uint8_t* ql = x[i].ql; const uint8_t* qh = x[i].qh; const int8_t* sc = x[i].scales;
      for (int n = 0; n < QK_K; n += 128) {
        for (int l = 0; l < 32; ++l) {
          const int is = l / 16;
          const int8_t q1 = (int8_t)((ql[l] & 0x0f) | (((qh[l] >> 0) & 3) << 4)) - 32;
          const int8_t q2 = (int8_t)((ql[l + 32] & 0x0f) | (((qh[l] >> 2) & 3) << 4)) - 32;
          const int8_t q3 = (int8_t)((ql[l] >> 4) | (((qh[l] >> 4) & 3) << 4)) - 32;
          const int8_t q4 = (int8_t)((ql[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4)) - 32;
          y[l + 0] = d * (float)sc[is + 0] * (float)q1;
          y[l + 32] = d * (float)sc[is + 2] * (float)q2;
          y[l + 64] = d * (float)sc[is + 4] * (float)q3;
          y[l + 96] = d * (float)sc[is + 6] * (float)q4;
        }
        y += 128; ql += 64; qh += 32; sc += 8;
      }
    }
    return 1;
  }
  return 0;
}

/* src/emel/kernel/detail.hpp:2846-2942 — same integers, same f32 order
 * (8 float lanes across blocks, min term in a separate running scalar) */
static float dot_q4_k_q8_k(const blk_q4_k* lhs, const blk_q8_k* rhs, uint64_t nblk) {
  float sums[8] = {0}; float sumf = 0.0f;
  int8_t aux8[QK_K]; int32_t aux32[8];
  for (uint64_t b = 0; b < nblk; ++b) {
    const uint8_t* q4 = lhs[b].qs; const int8_t* q8 = rhs[b].qs;
    int8_t* a = aux8;
    for (int g = 0; g < 4; ++g) {
      for (int l = 0; l < 32; ++l) a[l] = (int8_t)(q4[l] & 0x0f);
      a += 32;
      for (int l = 0; l < 32; ++l) a[l] = (int8_t)(q4[l] >> 4);
      a += 32; q4 += 32;
    }
    uint8_t sc[8], mn[8];
    for (int j = 0; j < 8; ++j) scale_min_k4(j, lhs[b].scales, &sc[j], &mn[j]);
    int32_t min_sum = 0;
    for (int g = 0; g < 16; ++g) min_sum += (int32_t)rhs[b].bsums[g] * (int32_t)mn[g / 2];
    memset(aux32, 0, sizeof aux32);
    a = aux8;
    for (int g = 0; g < 8; ++g) {
      const int32_t scale = sc[g];
      for (int strip = 0; strip < 4; ++strip) {
        for (int l = 0; l < 8; ++l) aux32[l] += scale * (int32_t)(int16_t)(q8[l] * a[l]);
        q8 += 8; a += 8;
      }
    }
    const float d = orc_fp16_to_fp32(lhs[b].d) * rhs[b].d;
    for (int l = 0; l < 8; ++l) sums[l] += d * (float)aux32[l];
    const float dmin = orc_fp16_to_fp32(lhs[b].dmin) * rhs[b].d;
    sumf -= dmin * (float)min_sum;
  }
  for (int l = 0; l < 8; ++l) sumf += sums[l];
  return sumf;
}

/* src/emel/kernel/detail.hpp:3062-3129 */
static float dot_q6_k_q8_k(const blk_q6_k* lhs, const blk_q8_k* rhs, uint64_t nblk) {
  float sums[8] = {0}; float sumf = 0.0f;
  int8_t aux8[QK_K]; int32_t aux32[8];
  for (uint64_t b = 0; b < nblk; ++b) {
    const uint8_t* q4 = lhs[b].ql; const uint8_t* qh = lhs[b].qh; const int8_t* q8 = rhs[b].qs;
    memset(aux32, 0, sizeof aux32);
    int8_t* a = aux8;
    for (int j = 0; j < QK_K; j += 128) {
      for (int l = 0; l < 32; ++l) {
        a[l + 0] = (int8_t)((q4[l] & 0x0f) | (((qh[l] >> 0) & 3) << 4)) - 32;
        a[l + 32] = (int8_t)((q4[l + 32] & 0x0f) | (((qh[l] >> 2) & 3) << 4)) - 32;
        a[l + 64] = (int8_t)((q4[l] >> 4) | (((qh[l] >> 4) & 3) << 4)) - 32;
        a[l + 96] = (int8_t)((q4[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4)) - 32;
      }
      a += 128; q4 += 64; qh += 32;
    }
    a = aux8;
    for (int g = 0; g < 16; ++g) {
      const int scale = lhs[b].scales[g];
      for (int strip = 0; strip < 2; ++strip) {
        for (int l = 0; l < 8; ++l) aux32[l] += scale * (int32_t)(int16_t)(q8[l] * a[l]);
        q8 += 8; a += 8;
      }
    }
    const float d = orc_fp16_to_fp32(lhs[b].d) * rhs[b].d;
    for (int l = 0; l < 8; ++l) sums[l] += d * (float)aux32[l];
  }
  for (int l = 0; l < 8; ++l) sumf += sums[l];
  return sumf;
}

/* src/emel/kernel/detail.hpp:3252-3269 */
static float dot_q8_0_q8_0(const blk_q8_0* lhs, const blk_q8_0* rhs, uint64_t nblk) {
  float sumf = 0.0f;
  for (uint64_t b = 0; b < nblk; ++b) {
    int32_t s = 0;
    for (int j = 0; j < 32; ++j) s += (int32_t)lhs[b].qs[j] * (int32_t)rhs[b].qs[j];
    sumf += (float)s * (orc_fp16_to_fp32(lhs[b].d) * orc_fp16_to_fp32(rhs[b].d));
  }
  return sumf;
}

/* src/emel/kernel/detail.hpp:3131-3153 */
static float dot_q4_0_q8_0(const blk_q4_0* lhs, const blk_q8_0* rhs, uint64_t nblk) {
  float sumf = 0.0f;
  for (uint64_t b = 0; b < nblk; ++b) {
    int32_t s0 = 0, s1 = 0;
    for (int j = 0; j < 16; ++j) {
      s0 += ((int32_t)(lhs[b].qs[j] & 0x0f) - 8) * (int32_t)rhs[b].qs[j];
      s1 += ((int32_t)(lhs[b].qs[j] >> 4) - 8) * (int32_t)rhs[b].qs[j + 16];
    }
    sumf += (float)(s0 + s1) * (orc_fp16_to_fp32(lhs[b].d) * orc_fp16_to_fp32(rhs[b].d));
  }
  return sumf;
}

float orc_row_dot(int type, const void* lhs, const void* rhs, uint64_t nblk) {
  switch (type) {
    case T_Q4_K: return dot_q4_k_q8_k((const blk_q4_k*)lhs, (const blk_q8_k*)rhs, nblk);
    case T_Q6_K: return dot_q6_k_q8_k((const blk_q6_k*)lhs, (const blk_q8_k*)rhs, nblk);
    case T_Q8_0: return dot_q8_0_q8_0((const blk_q8_0*)lhs, (const blk_q8_0*)rhs, nblk);
    case T_Q4_0: return dot_q4_0_q8_0((const blk_q4_0*)lhs, (const blk_q8_0*)rhs, nblk);
    default: return 0.0f;
  }
}

/* ---------- request validation ---------- */

static int is_k_type(int t) { return t == T_Q4_K || t == T_Q6_K; }
static int is_32_type(int t) { return t == T_Q4_0 || t == T_Q8_0; }
static int is_native_quant(int t) { return is_k_type(t) || is_32_type(t); }
static uint64_t block_elems(int t) { return is_k_type(t) ? QK_K : (is_32_type(t) ? 32 : 0); }
static uint64_t block_bytes(int t) {
  switch (t) { case T_Q4_0: return 18; case T_Q8_0: return 34; case T_Q4_K: return 144; case T_Q6_K: return 210; default: return 0; }
}
/* src/emel/kernel/detail.hpp:1545-1598: integer bytes per element, which
 * truncates to 0 for the sub-byte K-quants and Q4_0 */
static uint64_t elem_size(int t) {
  switch (t) { case T_F32: return 4; case T_F16: return 2; case T_Q8_0: return 34 / 32; case T_Q8_K: return 292 / 256;
    case T_Q4_0: return 18 / 32; case T_Q4_K: return 144 / 256; case T_Q6_K: return 210 / 256; default: return 0; }
}
static int is_supported(int t) { return t == T_F32 || t == T_F16 || is_native_quant(t) || t == T_Q8_K; }

/* src/emel/kernel/detail.hpp:1600-1697 */
uint64_t orc_row_bytes(int type, uint64_t cols) {
  const uint64_t be = block_elems(type);
  if (be == 0 || cols % be != 0) return 0;
  return cols / be * block_bytes(type);
}

/* src/emel/kernel/detail.hpp:1720-1737 */
static int valid_layout(const o_view* v) {
  const uint64_t es = elem_size(v->type);
  const int explicit_stride = v->nb[0] != 0;
  const int aligned = es != 0 && explicit_stride && v->nb[0] >= es && v->nb[0] % es == 0;
  int dims_ok = 1;
  for (int i = 0; i < 4; ++i) if (v->ne[i] > 1 && v->nb[i] == 0) dims_ok = 0;
  return es != 0 && (!explicit_stride || (aligned && dims_ok));
}
/* src/emel/kernel/detail.hpp:1709-1749 */
static uint64_t stride_bytes(const o_view* v, int dim) {
  uint64_t s = elem_size(v->type);
  for (int i = 0; i < dim; ++i) s *= v->ne[i];
  return v->nb[0] != 0 ? v->nb[dim] : s;
}
static int dense(const o_view* v) {
  uint64_t expect = elem_size(v->type);
  int ok = 1;
  for (int i = 0; i < 4; ++i) { ok = ok && stride_bytes(v, i) == expect; expect *= v->ne[i]; }
  return valid_layout(v) && ok;
}
static uint64_t elem_count(const o_view* v) { return v->ne[0] * v->ne[1] * v->ne[2] * v->ne[3]; }

/* src/emel/kernel/detail.hpp:1792-1927 restricted to the dtypes on this path */
static int required_src0_matmul(const o_view* s) {
  if (is_native_quant(s->type)) {
    const uint64_t rb = orc_row_bytes(s->type, s->ne[0]);
    return s->data && rb != 0 && s->ne[1] != 0 && s->ne[2] == 1 && s->ne[3] == 1 && s->nb[0] == 1 &&
           s->nb[1] == rb && s->nb[2] == rb * s->ne[1] && s->nb[3] == s->nb[2];
  }
  return s->data && is_supported(s->type) && valid_layout(s) && elem_count(s) > 0;
}
static int required_plain(const o_view* s) {
  return s->data && is_supported(s->type) && valid_layout(s) && elem_count(s) > 0;
}

/* src/emel/kernel/detail.hpp:3843-3872 (+ validate_dispatch_request 1919-1927);
 * f32×f32 matmul is accepted by the reference but is outside this path, so the
 * quantized predicate alone is restated */
int orc_can_run_mul_mat(const o_op* r) {
  if (!(required_src0_matmul(&r->src0) && required_plain(&r->src1) && required_plain(&r->dst))) return 0;
  if (r->op_params_size > 64) return 0;
  const uint64_t k = r->src0.ne[0], m = r->src0.ne[1], n = r->src1.ne[0];
  if (k == 0 || m == 0 || n == 0) return 0;
  const int shape = r->src1.ne[1] == k && r->dst.ne[0] == n && r->dst.ne[1] == m && r->src0.ne[2] == 1 &&
                    r->src0.ne[3] == 1 && r->src1.ne[2] == 1 && r->src1.ne[3] == 1 && r->dst.ne[2] == 1 && r->dst.ne[3] == 1;
  const int t = r->src0.type;
  const uint64_t be = block_elems(t);
  const uint64_t lim = is_32_type(t) ? MAX_Q8_0_BLOCKS : (is_k_type(t) ? MAX_Q8_K_BLOCKS : 0);
  const int q = is_native_quant(t) && r->src1.type == T_F32 && r->dst.type == T_F32 && be != 0 && k % be == 0 &&
                k / be <= lim && dense(&r->src1) && dense(&r->dst) && r->src0.nb[0] == 1 &&
                r->src0.nb[1] == orc_row_bytes(t, k) && r->src0.nb[2] == r->src0.nb[1] * m && r->src0.nb[3] == r->src0.nb[2];
  return shape && q;
}

/* src/emel/kernel/detail.hpp:3356-3571: for each token j, quantize column j of
 * src1 (element stride n), then one row dot per output row */
int orc_mul_mat(const o_op* r) {
  if (!orc_can_run_mul_mat(r)) return 0;
  const uint64_t k = r->src0.ne[0], m = r->src0.ne[1], n = r->src1.ne[0];
  const int t = r->src0.type;
  const float* b = (const float*)r->src1.data;
  float* c = (float*)r->dst.data;
  const uint8_t* a = (const uint8_t*)r->src0.data;
  const uint64_t rb = r->src0.nb[1];
  if (is_k_type(t)) {
    blk_q8_k* q8 = (blk_q8_k*)malloc(sizeof(blk_q8_k) * (k / QK_K));
    for (uint64_t j = 0; j < n; ++j) {
      orc_quantize_q8_k(b + j, n, q8, (int64_t)k);
      for (uint64_t i = 0; i < m; ++i) c[i * n + j] = orc_row_dot(t, a + i * rb, q8, k / QK_K);
    }
    free(q8);
  } else {
    blk_q8_0* q8 = (blk_q8_0*)malloc(sizeof(blk_q8_0) * (k / 32));
    for (uint64_t j = 0; j < n; ++j) {
      orc_quantize_q8_0(b + j, n, q8, (int64_t)k);
      for (uint64_t i = 0; i < m; ++i) c[i * n + j] = orc_row_dot(t, a + i * rb, q8, k / 32);
    }
    free(q8);
  }
  return 1;
}

/* src/emel/kernel/detail.hpp:3573-3731: strict > over ascending rows, so the
 * lowest row wins ties */
int orc_mul_mat_argmax(const o_op* r) {
  if (!(required_src0_matmul(&r->src0) && required_plain(&r->src1) && required_plain(&r->dst))) return 0;
  const uint64_t k = r->src0.ne[0], m = r->src0.ne[1], n = r->src1.ne[0];
  const int t = r->src0.type;
  const uint64_t be = block_elems(t);
  const uint64_t lim = is_32_type(t) ? MAX_Q8_0_BLOCKS : (is_k_type(t) ? MAX_Q8_K_BLOCKS : 0);
  const int shape = r->src1.ne[1] == k && r->dst.ne[0] == 1 && r->dst.ne[1] == 1 && r->src0.ne[2] == 1 && r->src0.ne[3] == 1 &&
                    r->src1.ne[2] == 1 && r->src1.ne[3] == 1 && r->dst.ne[2] == 1 && r->dst.ne[3] == 1;
  const int q = is_native_quant(t) && r->src1.type == T_F32 && r->dst.type == T_F32 && be != 0 && k % be == 0 && k / be <= lim &&
                dense(&r->src1) && dense(&r->dst) && r->src0.nb[0] == 1 && r->src0.nb[1] == orc_row_bytes(t, k) &&
                r->src0.nb[2] == r->src0.nb[1] * m && r->src0.nb[3] == r->src0.nb[2];
  if (k == 0 || m == 0 || n != 1 || !r->index_out || !shape || !q) return 0;
  /* run_mul_mat_argmax has branches for f32, Q5_0, Q8_0 and the K-quants only
   * (src/emel/kernel/detail.hpp:3621-3731): a Q4_0 request falls through to
   * `return false` although the guard accepts it */
  if (t == T_Q4_0) return 0;
  const float* b = (const float*)r->src1.data;
  const uint8_t* a = (const uint8_t*)r->src0.data;
  const uint64_t rb = r->src0.nb[1];
  void* q8 = malloc(is_k_type(t) ? sizeof(blk_q8_k) * (k / QK_K) : sizeof(blk_q8_0) * (k / 32));
  if (is_k_type(t)) orc_quantize_q8_k(b, 1, q8, (int64_t)k); else orc_quantize_q8_0(b, 1, q8, (int64_t)k);
  float best = -INFINITY; int32_t best_i = 0;
  for (uint64_t i = 0; i < m; ++i) {
    const float v = orc_row_dot(t, a + i * rb, q8, k / be);
    if (v > best || i == 0) { best = v; best_i = (int32_t)i; }
  }
  free(q8);
  *(float*)r->dst.data = best;
  *r->index_out = best_i;
  return 1;
}

/* ---------- flash decode attention ---------- */

/* src/emel/kernel/detail.hpp:4224-4252 */
static float fa_scale(const o_op* r) {
  if (r->op_params_size >= 4) { float s; memcpy(&s, r->op_params, 4); return s; }
  const float hd = (float)r->src0.ne[0];
  return hd > 0.0f ? 1.0f / sqrtf(hd) : 1.0f;
}
static uint64_t fa_masked_total(const o_op* r) {
  if (r->op_params_size >= 8) { uint32_t t; memcpy(&t, r->op_params + 4, 4); return t; }
  return r->src1.ne[1];
}

/* src/emel/kernel/detail.hpp:4346-4390 */
int orc_can_run_flash_attn(const o_op* r) {
  if (!(required_plain(&r->src0) && required_plain(&r->src1) && required_plain(&r->dst))) return 0;
  if (r->op_params_size > 64) return 0;
  const uint64_t hd = r->src0.ne[0], qc = r->src0.ne[1], hc = r->src0.ne[2], T = r->src1.ne[1], kvh = r->src1.ne[2];
  const int types = r->src0.type == T_F32 && r->src1.type == T_F16 && r->src2.type == T_F16 && r->dst.type == T_F32;
  const int dims = hd != 0 && qc == 1 && hc != 0 && T != 0 && kvh != 0;
  const int src2_ok = required_plain(&r->src2);
  const int shape = r->src1.ne[0] == hd && r->src2.ne[0] == hd && r->src2.ne[1] == T && r->src2.ne[2] == kvh &&
                    r->dst.ne[0] == hd && r->dst.ne[1] == qc && r->dst.ne[2] == hc && r->src0.ne[3] == 1 && r->src1.ne[3] == 1 &&
                    r->src2.ne[3] == 1 && r->dst.ne[3] == 1 && kvh != 0 && hc % (kvh ? kvh : 1) == 0;
  const int layout = dense(&r->src0) && valid_layout(&r->src1) && valid_layout(&r->src2) && dense(&r->dst);
  const float scale = fa_scale(r);
  return types && dims && src2_ok && shape && layout && fa_masked_total(r) >= T && isfinite(scale) && scale > 0.0f &&
         hd <= 4096; /* workspace bound, src/emel/kernel/detail.hpp:170, 5219-5227 */
}

static float round16(float v) { return orc_fp16_to_fp32(orc_fp32_to_fp16(v)); }

/* src/emel/kernel/detail.hpp:5238-5291 with dot_product_f16_f16_scores
 * (:2203-2208, f64 sum of exact f16 products), scale_f16_buffer_scalar
 * (:4312-4320) and axpy_f16_buffer_scalar (:4322-4332): sequential online
 * softmax, accumulator stored as f16 and rounded after every token */
int orc_flash_attn(const o_op* r) {
  if (!orc_can_run_flash_attn(r)) return 0;
  const uint64_t hd = r->src0.ne[0], hc = r->src0.ne[2], T = r->src1.ne[1], kvh = r->src1.ne[2];
  const float scale = fa_scale(r);
  const uint64_t n_rep = hc / kvh;
  uint16_t* qh = (uint16_t*)malloc(2 * hd);
  uint16_t* acc = (uint16_t*)malloc(2 * hd);
  for (uint64_t h = 0; h < hc; ++h) {
    const uint64_t kh = h / n_rep;
    const float* q = (const float*)((const char*)r->src0.data + h * r->src0.nb[2]);
    float* dst = (float*)((char*)r->dst.data + h * r->dst.nb[2]);
    for (uint64_t i = 0; i < hd; ++i) { qh[i] = orc_fp32_to_fp16(q[i]); acc[i] = 0; }
    float sum = 0.0f, mx = -INFINITY;
    for (uint64_t t = 0; t < T; ++t) {
      const uint16_t* kk = (const uint16_t*)((const char*)r->src1.data + t * r->src1.nb[1] + kh * r->src1.nb[2]);
      const uint16_t* vv = (const uint16_t*)((const char*)r->src2.data + t * r->src2.nb[1] + kh * r->src2.nb[2]);
      double s = 0.0;
      for (uint64_t i = 0; i < hd; ++i) s += (double)orc_fp16_to_fp32(qh[i]) * (double)orc_fp16_to_fp32(kk[i]);
      const float score = (float)s * scale;
      const float old = mx;
      float ms = 1.0f, vs = 1.0f;
      if (score > mx) {
        mx = score;
        ms = expf(old - mx);
        const float rs = round16(ms);
        for (uint64_t i = 0; i < hd; ++i) acc[i] = orc_fp32_to_fp16(round16(orc_fp16_to_fp32(acc[i]) * rs));
      } else {
        vs = expf(score - mx);
      }
      const float ra = round16(vs);
      for (uint64_t i = 0; i < hd; ++i)
        acc[i] = orc_fp32_to_fp16(round16(orc_fp16_to_fp32(acc[i]) + orc_fp16_to_fp32(vv[i]) * ra));
      sum = sum * ms + vs;
    }
    if (sum == 0.0f) { for (uint64_t i = 0; i < hd; ++i) dst[i] = 0.0f; }
    else { const float inv = 1.0f / sum; for (uint64_t i = 0; i < hd; ++i) dst[i] = orc_fp16_to_fp32(acc[i]) * inv; }
  }
  free(qh); free(acc);
  return 1;
}

/* f64 softmax attention over the same f16 inputs: ground truth used to show
 * which side of a tolerance carries the error (no reference counterpart) */
int orc_flash_attn_f64(const o_op* r, double* out) {
  if (!orc_can_run_flash_attn(r)) return 0;
  const uint64_t hd = r->src0.ne[0], hc = r->src0.ne[2], T = r->src1.ne[1], kvh = r->src1.ne[2];
  const double scale = (double)fa_scale(r);
  const uint64_t n_rep = hc / kvh;
  double* s = (double*)malloc(sizeof(double) * T);
  for (uint64_t h = 0; h < hc; ++h) {
    const uint64_t kh = h / n_rep;
    const float* q = (const float*)((const char*)r->src0.data + h * r->src0.nb[2]);
    double mx = -INFINITY;
    for (uint64_t t = 0; t < T; ++t) {
      const uint16_t* kk = (const uint16_t*)((const char*)r->src1.data + t * r->src1.nb[1] + kh * r->src1.nb[2]);
      double a = 0.0;
      for (uint64_t i = 0; i < hd; ++i) a += (double)round16(q[i]) * (double)orc_fp16_to_fp32(kk[i]);
      s[t] = a * scale; if (s[t] > mx) mx = s[t];
    }
    double den = 0.0;
    for (uint64_t t = 0; t < T; ++t) { s[t] = exp(s[t] - mx); den += s[t]; }
    for (uint64_t i = 0; i < hd; ++i) {
      double a = 0.0;
      for (uint64_t t = 0; t < T; ++t) {
        const uint16_t* vv = (const uint16_t*)((const char*)r->src2.data + t * r->src2.nb[1] + kh * r->src2.nb[2]);
        a += s[t] * (double)orc_fp16_to_fp32(vv[i]);
      }
      out[h * hd + i] = a / den;
    }
  }
  free(s);
  return 1;
}

/* ---------- row slicing ---------- */

/* src/emel/kernel/matmul/actions.hpp:48-67 with group_rows = 1 (native rows) */
void orc_row_slice(uint64_t rows, uint32_t lane, uint32_t lane_count, uint64_t* begin, uint64_t* count) {
  const uint64_t per = rows / lane_count, extra = rows % lane_count;
  *begin = lane * per + (lane < extra ? lane : extra);
  *count = per + (lane < extra ? 1u : 0u);
}

/* ---------- own-design weight encoders (no reference counterpart) ---------- */

/* Q4_K: per 32-element sub-block an affine 4-bit code (min clipped to <= 0),
 * sub-block scale/min then coded in 6 bits against per-super-block f16 d/dmin.
 * Decodes through orc_dequantize_row / the reference decoder unchanged. */
void orc_encode_q4_k(const float* x, void* out, int64_t k) {
  blk_q4_k* y = (blk_q4_k*)out;
  for (int64_t i = 0; i < k / QK_K; ++i) {
    const float* xb = x + i * QK_K;
    float sc[8], mn[8];
    float max_sc = 0.0f, max_mn = 0.0f;
    for (int j = 0; j < 8; ++j) {
      float lo = xb[j * 32], hi = xb[j * 32];
      for (int l = 1; l < 32; ++l) { const float v = xb[j * 32 + l]; if (v < lo) lo = v; if (v > hi) hi = v; }
      if (lo > 0.0f) lo = 0.0f;
      sc[j] = (hi - lo) / 15.0f;
      mn[j] = -lo;
      if (sc[j] > max_sc) max_sc = sc[j];
      if (mn[j] > max_mn) max_mn = mn[j];
    }
    const float d = max_sc / 63.0f, dm = max_mn / 63.0f;
    y[i].d = orc_fp32_to_fp16(d);
    y[i].dmin = orc_fp32_to_fp16(dm);
    const float dq = orc_fp16_to_fp32(y[i].d), dmq = orc_fp16_to_fp32(y[i].dmin);
    uint8_t ls[8], lm[8];
    for (int j = 0; j < 8; ++j) {
      int a = dq > 0.0f ? (int)lrintf(sc[j] / dq) : 0;
      int b = dmq > 0.0f ? (int)lrintf(mn[j] / dmq) : 0;
      ls[j] = (uint8_t)(a < 0 ? 0 : (a > 63 ? 63 : a));
      lm[j] = (uint8_t)(b < 0 ? 0 : (b > 63 ? 63 : b));
    }
    memset(y[i].scales, 0, 12);
    for (int j = 0; j < 8; ++j) {
      if (j < 4) { y[i].scales[j] = ls[j]; y[i].scales[j + 4] = lm[j]; }
      else {
        y[i].scales[j + 4] = (uint8_t)((ls[j] & 0x0f) | ((lm[j] & 0x0f) << 4));
        y[i].scales[j - 4] |= (uint8_t)((ls[j] >> 4) << 6);
        y[i].scales[j] |= (uint8_t)((lm[j] >> 4) << 6);
      }
    }
    for (int g = 0; g < 4; ++g) {
      const float d0 = dq * (float)ls[2 * g], m0 = dmq * (float)lm[2 * g];
      const float d1 = dq * (float)ls[2 * g + 1], m1 = dmq * (float)lm[2 * g + 1];
      for (int l = 0; l < 32; ++l) {
        int a = d0 > 0.0f ? (int)lrintf((xb[g * 64 + l] + m0) / d0) : 0;
        int b = d1 > 0.0f ? (int)lrintf((xb[g * 64 + 32 + l] + m1) / d1) : 0;
        a = a < 0 ? 0 : (a > 15 ? 15 : a);
        b = b < 0 ? 0 : (b > 15 ? 15 : b);
        y[i].qs[g * 32 + l] = (uint8_t)(a | (b << 4));
      }
    }
  }
}

/* Q6_K: per 16-element group a symmetric 6-bit code; group scales coded as
 * int8 against the per-super-block f16 d. */
void orc_encode_q6_k(const float* x, void* out, int64_t k) {
  blk_q6_k* y = (blk_q6_k*)out;
  for (int64_t i = 0; i < k / QK_K; ++i) {
    const float* xb = x + i * QK_K;
    float gs[16]; float max_abs_scale = 0.0f;
    for (int g = 0; g < 16; ++g) {
      float amax = 0.0f;
      for (int l = 0; l < 16; ++l) { const float a = fabsf(xb[g * 16 + l]); if (a > amax) amax = a; }
      gs[g] = amax / 31.0f;
      if (gs[g] > max_abs_scale) max_abs_scale = gs[g];
    }
    const float d = max_abs_scale / 127.0f;
    y[i].d = orc_fp32_to_fp16(d);
    const float dq = orc_fp16_to_fp32(y[i].d);
    int8_t q[QK_K];
    for (int g = 0; g < 16; ++g) {
      int s = dq > 0.0f ? (int)lrintf(gs[g] / dq) : 0;
      if (s > 127) s = 127;
      if (s < 1 && gs[g] > 0.0f) s = 1;
      y[i].scales[g] = (int8_t)s;
      const float step = dq * (float)s;
      for (int l = 0; l < 16; ++l) {
        int v = step > 0.0f ? (int)lrintf(xb[g * 16 + l] / step) : 0;
        v = v < -32 ? -32 : (v > 31 ? 31 : v);
        q[g * 16 + l] = (int8_t)(v + 32);
      }
    }
    for (int n = 0; n < 2; ++n) {
      for (int l = 0; l < 32; ++l) {
        const uint8_t q1 = (uint8_t)q[n * 128 + l], q2 = (uint8_t)q[n * 128 + l + 32];
        const uint8_t q3 = (uint8_t)q[n * 128 + l + 64], q4 = (uint8_t)q[n * 128 + l + 96];
        y[i].ql[n * 64 + l] = (uint8_t)((q1 & 0x0f) | ((q3 & 0x0f) << 4));
        y[i].ql[n * 64 + l + 32] = (uint8_t)((q2 & 0x0f) | ((q4 & 0x0f) << 4));
        y[i].qh[n * 32 + l] = (uint8_t)((q1 >> 4) | ((q2 >> 4) << 2) | ((q3 >> 4) << 4) | ((q4 >> 4) << 6));
      }
    }
  }
}

/* encode a whole {K, M} matrix row by row; Q8_0 weights go through the
 * reference-owned activation quantizer (stride 1), Q4_0 through its own
 * reference encoder */
int orc_encode_rows(int type, const float* x, void* out, uint64_t k, uint64_t m) {
  const uint64_t rb = orc_row_bytes(type, k);
  if (rb == 0) return 0;
  for (uint64_t i = 0; i < m; ++i) {
    uint8_t* dst = (uint8_t*)out + i * rb;
    const float* src = x + i * k;
    switch (type) {
      case T_Q4_K: orc_encode_q4_k(src, dst, (int64_t)k); break;
      case T_Q6_K: orc_encode_q6_k(src, dst, (int64_t)k); break;
      case T_Q8_0: orc_quantize_q8_0(src, 1, dst, (int64_t)k); break;
      case T_Q4_0: orc_quantize_q4_0(src, dst, (int64_t)k); break;
      default: return 0;
    }
  }
  return 1;
}
