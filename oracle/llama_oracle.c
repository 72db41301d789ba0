/*
 * TEST INFRASTRUCTURE ONLY — CPU restatement of the reference generator's
 * per-token decode loop for a Llama-architecture model, used to check the
 * device-resident decoder.  Never linked into or called by the product path.
 *
 * The reference's own loop (src/emel/text/generator/detail.hpp) cannot be
 * compiled here: it includes the un-vendored state-machine library.  Its layer
 * math is restated below; every matrix product and every attention call goes
 * through function pointers, so the caller can plug in either the plain-C
 * kernels of emel_oracle.c or the reference's own kernels from oracle/_ref.
 *
 *   rms_norm                          detail.hpp:2735-2756
 *   apply_rope_pairing                detail.hpp:2905-2936
 *   silu                              detail.hpp:2967-2973
 *   store_attention_kv_cache          detail.hpp:3294-3332 (flash layout :3010-3048)
 *   make_flash_attn_request           detail.hpp:3232-3279
 *   compute_layer_attention_residual  detail.hpp:3746-3840
 *   compute_layer_feed_forward        detail.hpp:3852-3926
 *   compute_logits                    detail.hpp:3997-4033
 *   run_decode                        detail.hpp:4860-4914
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

typedef struct { const void* data; uint8_t type; uint64_t ne[4]; uint64_t nb[4]; } o_view;
typedef struct { o_view src0, src1, src2, dst; uint8_t op_params[64]; uint32_t op_params_size; int32_t* index_out; } o_op;

uint16_t orc_fp32_to_fp16(float f);
uint64_t orc_row_bytes(int type, uint64_t cols);
int orc_dequantize_row(int type, const void* src, float* y, int64_t k);

typedef int (*mul_mat_fn)(const o_op*);
typedef int (*flash_fn)(const o_op*);

typedef struct {
  const void* data;
  int32_t type;
} l_tensor;

typedef struct {
  int32_t n_layer, n_embd, n_head, n_head_kv, head_dim, n_ff, n_vocab, n_ctx, rope_dim, rope_neox, kv_block;
  float rope_freq_base, rms_eps;
} l_config;

typedef struct {
  l_config cfg;
  l_tensor tok_embd, out_norm, output;
  l_tensor* layers; /* 9 per layer: attn_norm, wq, wk, wv, wo, ffn_norm, gate, up, down */
  mul_mat_fn mul_mat;
  flash_fn flash;
  int64_t capacity;
  uint16_t *kcache, *vcache;
  float *hidden, *norm, *q, *k, *v, *attn, *gate, *up, *ffn, *proj;
} l_model;

static void rms_norm(const float* x, const float* w, float eps, int n, float* out) {
  double ss = 0.0;
  for (int i = 0; i < n; ++i) ss += (double)(x[i] * x[i]);
  const float mean = (float)(ss / (double)n);
  const float scale = 1.0f / sqrtf(mean + eps);
  for (int i = 0; i < n; ++i) { out[i] = x[i]; out[i] *= scale; out[i] *= w[i]; }
}

static void rope(float* vec, int heads, int head_dim, int n_rot, int neox, int position, float base) {
  const int rot = n_rot < head_dim ? n_rot : head_dim;
  if (heads <= 0 || head_dim <= 1 || rot <= 1) return;
  const float theta_scale = powf(base, -2.0f / (float)rot);
  const int pairs = rot / 2;
  const int x0s = neox ? 1 : 2, x1s = neox ? 1 : 2, x1b = neox ? pairs : 1;
  for (int h = 0; h < heads; ++h) {
    float* p = vec + (size_t)h * head_dim;
    float theta = (float)position;
    for (int i = 0; i < pairs; ++i) {
      const float c = cosf(theta), s = sinf(theta);
      const int d0 = i * x0s, d1 = i * x1s + x1b;
      const float x0 = p[d0], x1 = p[d1];
      p[d0] = x0 * c - x1 * s;
      p[d1] = x0 * s + x1 * c;
      theta *= theta_scale;
    }
  }
}

static void fill_view_quant(o_view* v, const l_tensor* t, uint64_t k, uint64_t m) {
  const uint64_t rb = orc_row_bytes(t->type, k);
  v->data = t->data; v->type = (uint8_t)t->type;
  v->ne[0] = k; v->ne[1] = m; v->ne[2] = 1; v->ne[3] = 1;
  v->nb[0] = 1; v->nb[1] = rb; v->nb[2] = rb * m; v->nb[3] = rb * m;
}
static void fill_view_f32(o_view* v, const void* data, uint64_t n0, uint64_t n1, uint64_t n2) {
  v->data = data; v->type = 0;
  v->ne[0] = n0; v->ne[1] = n1; v->ne[2] = n2; v->ne[3] = 1;
  v->nb[0] = 4; v->nb[1] = 4 * n0; v->nb[2] = 4 * n0 * n1; v->nb[3] = 4 * n0 * n1 * n2;
}

/* matmul_vector, detail.hpp:2290-2314: src1 = f32 {1, K}, dst = f32 {1, M} */
static int matvec(const l_model* m, const l_tensor* w, int K, int M, const float* x, float* y) {
  o_op op; memset(&op, 0, sizeof op);
  fill_view_quant(&op.src0, w, (uint64_t)K, (uint64_t)M);
  fill_view_f32(&op.src1, x, 1, (uint64_t)K, 1);
  fill_view_f32(&op.dst, y, 1, (uint64_t)M, 1);
  return m->mul_mat(&op);
}

l_model* orc_llama_create(const l_config* cfg, mul_mat_fn mm, flash_fn fa) {
  l_model* m = (l_model*)calloc(1, sizeof(l_model));
  m->cfg = *cfg;
  m->mul_mat = mm;
  m->flash = fa;
  m->layers = (l_tensor*)calloc((size_t)cfg->n_layer * 9, sizeof(l_tensor));
  const int kvb = cfg->kv_block > 0 ? cfg->kv_block : 16;
  m->capacity = ((int64_t)cfg->n_ctx + kvb - 1) / kvb * kvb;
  const size_t cache = (size_t)cfg->n_layer * cfg->n_head_kv * (size_t)m->capacity * cfg->head_dim;
  m->kcache = (uint16_t*)calloc(cache, 2);
  m->vcache = (uint16_t*)calloc(cache, 2);
  const size_t qd = (size_t)cfg->n_head * cfg->head_dim, kvd = (size_t)cfg->n_head_kv * cfg->head_dim;
  m->hidden = (float*)calloc(cfg->n_embd, 4); m->norm = (float*)calloc(cfg->n_embd, 4);
  m->proj = (float*)calloc(cfg->n_embd, 4);
  m->q = (float*)calloc(qd, 4); m->attn = (float*)calloc(qd, 4);
  m->k = (float*)calloc(kvd, 4); m->v = (float*)calloc(kvd, 4);
  m->gate = (float*)calloc(cfg->n_ff, 4); m->up = (float*)calloc(cfg->n_ff, 4); m->ffn = (float*)calloc(cfg->n_ff, 4);
  return m;
}

void orc_llama_destroy(l_model* m) {
  if (!m) return;
  free(m->layers); free(m->kcache); free(m->vcache); free(m->hidden); free(m->norm); free(m->proj);
  free(m->q); free(m->attn); free(m->k); free(m->v); free(m->gate); free(m->up); free(m->ffn);
  free(m);
}

/* role numbering of include/emelb_llama.h */
int orc_llama_bind(l_model* m, int layer, int role, const void* data, int type) {
  l_tensor t = {data, type};
  if (role == 0) m->tok_embd = t;
  else if (role == 1) m->out_norm = t;
  else if (role == 2) m->output = t;
  else if (role >= 3 && role <= 11 && layer >= 0 && layer < m->cfg.n_layer) m->layers[(size_t)layer * 9 + (role - 3)] = t;
  else return 0;
  return 1;
}

/* one token; logits (n_vocab) may be null to skip compute_logits (prefill) */
int orc_llama_decode(l_model* m, int token, int position, float* logits) {
  const l_config* c = &m->cfg;
  if (token < 0 || token >= c->n_vocab || position < 0 || position >= c->n_ctx) return 0;
  const int qd = c->n_head * c->head_dim, kvd = c->n_head_kv * c->head_dim;
  /* copy_tensor_row: dequantize the embedding row */
  if (m->tok_embd.type == 0) {
    memcpy(m->hidden, (const float*)m->tok_embd.data + (size_t)token * c->n_embd, 4 * (size_t)c->n_embd);
  } else {
    const uint64_t rb = orc_row_bytes(m->tok_embd.type, (uint64_t)c->n_embd);
    if (!orc_dequantize_row(m->tok_embd.type, (const uint8_t*)m->tok_embd.data + (size_t)token * rb, m->hidden, c->n_embd)) return 0;
  }
  for (int l = 0; l < c->n_layer; ++l) {
    const l_tensor* w = m->layers + (size_t)l * 9;
    rms_norm(m->hidden, (const float*)w[0].data, c->rms_eps, c->n_embd, m->norm);
    if (!matvec(m, &w[1], c->n_embd, qd, m->norm, m->q)) return 0;
    if (!matvec(m, &w[2], c->n_embd, kvd, m->norm, m->k)) return 0;
    if (!matvec(m, &w[3], c->n_embd, kvd, m->norm, m->v)) return 0;
    rope(m->q, c->n_head, c->head_dim, c->rope_dim, c->rope_neox, position, c->rope_freq_base);
    rope(m->k, c->n_head_kv, c->head_dim, c->rope_dim, c->rope_neox, position, c->rope_freq_base);
    const size_t layer_off = (size_t)l * c->n_head_kv * (size_t)m->capacity * c->head_dim;
    for (int h = 0; h < c->n_head_kv; ++h) {
      uint16_t* kd = m->kcache + layer_off + ((size_t)h * m->capacity + position) * c->head_dim;
      uint16_t* vd = m->vcache + layer_off + ((size_t)h * m->capacity + position) * c->head_dim;
      for (int d = 0; d < c->head_dim; ++d) {
        kd[d] = orc_fp32_to_fp16(m->k[(size_t)h * c->head_dim + d]);
        vd[d] = orc_fp32_to_fp16(m->v[(size_t)h * c->head_dim + d]);
      }
    }
    {
      o_op op; memset(&op, 0, sizeof op);
      const uint64_t T = (uint64_t)position + 1, hd = (uint64_t)c->head_dim;
      fill_view_f32(&op.src0, m->q, hd, 1, (uint64_t)c->n_head);
      o_view* kv[2] = {&op.src1, &op.src2};
      const uint16_t* base[2] = {m->kcache + layer_off, m->vcache + layer_off};
      for (int i = 0; i < 2; ++i) {
        kv[i]->data = base[i]; kv[i]->type = 1;
        kv[i]->ne[0] = hd; kv[i]->ne[1] = T; kv[i]->ne[2] = (uint64_t)c->n_head_kv; kv[i]->ne[3] = 1;
        kv[i]->nb[0] = 2; kv[i]->nb[1] = 2 * hd; kv[i]->nb[2] = 2 * (uint64_t)m->capacity * hd;
        kv[i]->nb[3] = kv[i]->nb[2] * (uint64_t)c->n_head_kv;
      }
      fill_view_f32(&op.dst, m->attn, hd, 1, (uint64_t)c->n_head);
      const float scale = 1.0f / sqrtf((float)c->head_dim);
      const uint32_t masked = (uint32_t)c->n_ctx;
      memcpy(op.op_params, &scale, 4); memcpy(op.op_params + 4, &masked, 4);
      op.op_params_size = 8;
      if (!m->flash(&op)) return 0;
    }
    if (!matvec(m, &w[4], qd, c->n_embd, m->attn, m->proj)) return 0;
    for (int i = 0; i < c->n_embd; ++i) m->hidden[i] += m->proj[i];
    rms_norm(m->hidden, (const float*)w[5].data, c->rms_eps, c->n_embd, m->norm);
    if (!matvec(m, &w[6], c->n_embd, c->n_ff, m->norm, m->gate)) return 0;
    if (!matvec(m, &w[7], c->n_embd, c->n_ff, m->norm, m->up)) return 0;
    for (int i = 0; i < c->n_ff; ++i) m->ffn[i] = (m->gate[i] / (1.0f + expf(-m->gate[i]))) * m->up[i];
    if (!matvec(m, &w[8], c->n_ff, c->n_embd, m->ffn, m->proj)) return 0;
    for (int i = 0; i < c->n_embd; ++i) m->hidden[i] += m->proj[i];
  }
  if (!logits) return 1;
  rms_norm(m->hidden, (const float*)m->out_norm.data, c->rms_eps, c->n_embd, m->norm);
  return matvec(m, &m->output, c->n_embd, c->n_vocab, m->norm, logits);
}

/* element-wise pieces exported on their own, for kernel-level checks */
void orc_rms_norm(const float* x, const float* w, float eps, int n, float* out) { rms_norm(x, w, eps, n, out); }
void orc_rope(float* vec, int heads, int head_dim, int n_rot, int neox, int position, float base) {
  rope(vec, heads, head_dim, n_rot, neox, position, base);
}
void orc_swiglu(const float* gate, const float* up, int n, float* out) {
  for (int i = 0; i < n; ++i) out[i] = (gate[i] / (1.0f + expf(-gate[i]))) * up[i];
}
