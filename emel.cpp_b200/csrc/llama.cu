// Device-resident decode loop (include/emelb_llama.h): the reference
// generator's per-token call sequence restated over this library's kernels.
//   run_decode                         src/emel/text/generator/detail.hpp:4860-4914
//   compute_layer_attention_residual   :3746-3840
//   compute_layer_feed_forward         :3852-3926
//   compute_logits                     :3997-4033
// One token step is a fixed chain of kernels whose token id, position and KV
// length live in device memory, so the chain is captured once as a CUDA graph
// and replayed per token.
//
// Row sharding (shard_count = G > 1, one process per GPU): rank r holds rows
// [r*M/G, (r+1)*M/G) of every matrix, which for Q/K/V means n_head/G query heads
// and n_head_kv/G KV heads, so the KV cache and attention are local.  Four f32
// all-gathers per layer join the row intervals (attention context, hidden after
// the output projection, the SwiGLU product, hidden after the down projection);
// every vector that gets quantized is the full, identical vector on every rank,
// so the token stream equals the unsharded one bit for bit — the contract the
// reference's row-slice fork/join keeps across lane counts
// (src/emel/kernel/matmul/detail.hpp:36-57).
#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <new>
#include <vector>

#include "../../include/emelb_llama.h"
#include "../../include/emelb_window.h"
#include "ctx.h"
#include "window.h"

using namespace emelb;

namespace emelb {
const void* ctx_resolve_weights(emelb_ctx* c, const void* p);  // api.cu
bool ctx_cuda_ok(emelb_ctx* c, cudaError_t e);
cudaError_t comm_all_gather_bytes(emelb_ctx* c, void* buf, size_t bytes_per_rank, cudaStream_t st);  // comm.cu
}  // namespace emelb

namespace {

struct Tensor {
  const uint8_t* dev = nullptr;
  int64_t win_off = -1;   // >= 0: the tensor is streamed; its offset inside the layer's slot of the session's window
  int type = EMELB_UNKNOWN;
  int64_t row_bytes = 0;
  int K = 0, M = 0;
};

struct Layer {
  Tensor attn_norm, wq, wk, wv, wo, ffn_norm, gate, up, down;
};

enum Mode { MODE_PREFILL = 0, MODE_LOGITS = 1, MODE_ARGMAX = 2, MODE_COUNT = 3 };

int family_of(int type) { return is_k_type(type) ? 1 : 2; }

}  // namespace

struct emelb_llama {
  emelb_ctx* c = nullptr;
  emelb_llama_config cfg{};
  std::vector<Layer> layers;
  Tensor tok_embd, out_norm, output;
  int64_t capacity = 0;
  // activations (f32, device)
  float *hidden = nullptr, *norm = nullptr, *q = nullptr, *k = nullptr, *v = nullptr, *attn = nullptr;
  float *gate = nullptr, *up = nullptr, *ffn = nullptr, *logits = nullptr;
  __half *kcache = nullptr, *vcache = nullptr;
  float *rope_cos = nullptr, *rope_sin = nullptr;
  int* state = nullptr;       // {token, position, kv_tokens, step}
  int* tokens_dev = nullptr;  // generated ids (n_ctx)
  int* host_pinned = nullptr;
  // token-batch buffers of the prompt path (feature-major {features, batch}), allocated by the first batched prefill
  int batch_cap = 0;
  int* batch_tokens = nullptr;
  float *b_hidden = nullptr, *b_norm = nullptr, *b_q = nullptr, *b_k = nullptr, *b_v = nullptr, *b_attn = nullptr;
  float *b_gate = nullptr, *b_up = nullptr, *b_ffn = nullptr, *b_y = nullptr;
  double* b_partial = nullptr;
  int fa_splits = 1;
  // sequences decoded together (emelb_llama_set_sequences): the cache planes are [layer][sequence][kv head][capacity][d];
  // the one-sequence entry points work on sequence cur_seq
  int n_seq = 1, cur_seq = 0;
  int* bstate = nullptr;      // rows of kMaxSeqs ints: token, position, kv token count; then {step}
  int* b_idx = nullptr;       // next token per sequence
  int* b_out = nullptr;       // generated ids, [step][sequence]
  float *b_qs = nullptr, *b_logits = nullptr, *b_part_acc = nullptr, *b_part_ml = nullptr, *b_amax_val = nullptr;
  int* b_amax_idx = nullptr;
  int seq_cap = 0;            // sequences the batch-step buffers were sized for
  cudaGraphExec_t batch_graph = nullptr;
  int batch_graph_B = 0, batch_graph_mode = -1, batch_launches = 0;
  int G = 1, rank = 0;        // row sharding
  int* pair_buf = nullptr;    // G x 16-byte records {value bits, global row, -, -}: argmax candidates
  // sharded sessions keep the vectors that are joined across ranks in one allocation (the exchange arena) so
  // peers can map it; with every peer attached the joins run as peer stores instead of NCCL calls
  char* arena = nullptr;
  size_t arena_bytes = 0, flags_off = 0, seq_off = 0;
  ActPlanesMut attn_planes{}, ffn_planes{};   // Q8_K planes of the joined attention context / SwiGLU product (in the arena)
  char* peer_base[kMaxPeers] = {};
  bool peers_attached = false;
  // peers attached: joins inside the producing / consuming kernels where a layer qualifies.  Opt-in: measured equal to
  // one join kernel each on 2 GPUs and 10 % slower on 4
  bool fused_joins = false;
  // descriptors of the fused joins in device memory, written when the peers are attached: [join id] (0 unused)
  JoinOut* join_out_dev = nullptr;
  JoinIn* join_in_dev = nullptr;    // peers attached: joins inside the producing / consuming kernels where a layer qualifies
  cudaGraphExec_t graphs[MODE_COUNT] = {nullptr, nullptr, nullptr};
  int graph_attention_mode[MODE_COUNT] = {-1, -1, -1};
  int launches_per_token = 0;          // of the argmax step
  int launches_mode[MODE_COUNT] = {0, 0, 0};
  // which f32 vector the context's activation planes currently hold, and for which family
  const float* planes_src = nullptr;
  int planes_family = 0;
  // whole-token kernel (token_kernel.cu): the layers' weight pointers as a device array, rebuilt after a bind
  TokenLayerW* token_layers = nullptr;
  bool token_layers_valid = false;
  bool token_usable = false;     // the model's shapes and types fit that kernel
  // prompt tokens per batch (0: walk the prompt token by token).  2048 gives 64 to 224 weight-row x token tiles
  // per product at the 8B shape: the tensor-core kernel's grid fills
  int prefill_batch = 2048;
  int step_mode = 0;             // 0: the chain of per-operation launches, 1: one kernel per token where it applies
  TokenLaunchState token_launch;
  unsigned long long* token_trace = nullptr;   // device stamps of emelb_llama_decode_profile
  // a streaming layer window (emelb_llama_set_window): layer tensors bound to addresses inside its source are read
  // from the slot the window hands out for the layer; steps then run as plain launches, not as replayed graphs
  emelb_window* window = nullptr;
  bool streamed = false;
  std::vector<void*> owned;
};

namespace {

constexpr int kMaxSeqs = 64;

// offset (halves) of sequence seq's planes of layer l inside the K or V cache
int64_t cache_off(const emelb_llama* s, int l, int seq) {
  return ((int64_t)l * s->n_seq + seq) * (s->cfg.n_head_kv / s->G) * s->capacity * s->cfg.head_dim;
}

bool dev_alloc(emelb_llama* s, void** p, size_t bytes) {
  if (cudaMalloc(p, (bytes + 255) & ~size_t(255)) != cudaSuccess) {
    cudaGetLastError();
    return false;
  }
  s->owned.push_back(*p);
  return true;
}

bool bound(const Tensor& t) { return t.dev != nullptr || t.win_off >= 0; }

// layer tensors that are streamed through the session's window instead of being resident
int streamed_tensors(const emelb_llama* s) {
  int n = 0;
  for (const Layer& l : s->layers)
    for (const Tensor* t : {&l.attn_norm, &l.wq, &l.wk, &l.wv, &l.wo, &l.ffn_norm, &l.gate, &l.up, &l.down}) n += t->win_off >= 0;
  return n;
}

bool all_bound(const emelb_llama* s) {
  if (!bound(s->tok_embd) || !bound(s->out_norm) || !bound(s->output)) return false;
  for (const Layer& l : s->layers)
    if (!(bound(l.attn_norm) && bound(l.wq) && bound(l.wk) && bound(l.wv) && bound(l.wo) && bound(l.ffn_norm) &&
          bound(l.gate) && bound(l.up) && bound(l.down)))
      return false;
  return true;
}

TokenArgs token_args(emelb_llama* s) {
  const emelb_llama_config& c = s->cfg;
  TokenArgs a{};
  a.layers = s->token_layers;
  a.n_layer = c.n_layer;
  a.n_embd = c.n_embd;
  a.n_ff = c.n_ff;
  a.heads = c.n_head;
  a.kv_heads = c.n_head_kv;
  a.head_dim = c.head_dim;
  a.eps = c.rms_eps;
  a.state = s->state;
  a.hidden = s->hidden;
  a.q = s->q;
  a.ffn = s->ffn;
  a.attn_planes = ActPlanesMut{s->c->act_qs, s->c->act_d, s->c->act_bsums};
  a.attn_f32 = nullptr;
  a.kcache = s->kcache;
  a.vcache = s->vcache;
  a.capacity = s->capacity;
  a.rope_cos = s->rope_cos;
  a.rope_sin = s->rope_sin;
  a.rope_rot_dim = c.rope_dim < c.head_dim ? c.rope_dim : c.head_dim;
  a.attn_scale = 1.0f / std::sqrt((float)c.head_dim);
  a.fa_splits = s->fa_splits;
  a.part_acc = s->c->fa_part_acc;
  a.part_ml = s->c->fa_part_ml;
  a.kv_cnt = s->c->token_cnt;
  a.bv_table = s->c->bv_table;
  a.grp_cnt = s->c->grp_cnt;
  a.bar = s->c->token_bar;
  a.status = s->c->status_word();
  a.trace = nullptr;
  return a;
}

// Whether one decode token of this session can run as the single persistent kernel, and its device-side layer
// table (uploaded here, outside any capture).  The kernel takes unsharded sessions whose layer matrices are all
// Q4_K with 16-byte aligned rows, adjacent-pair RoPE and the fast attention.
void prepare_token_kernel(emelb_llama* s) {
  if (s->token_layers_valid) return;
  s->token_layers_valid = true;
  s->token_usable = false;
  const emelb_llama_config& c = s->cfg;
  if (s->G != 1 || c.rope_neox || (c.head_dim & 1) || !all_bound(s) || s->streamed) return;
  std::vector<TokenLayerW> host(c.n_layer);
  for (int l = 0; l < c.n_layer; ++l) {
    const Layer& w = s->layers[l];
    const Tensor* mats[7] = {&w.wq, &w.wk, &w.wv, &w.wo, &w.gate, &w.up, &w.down};
    for (const Tensor* t : mats)
      if (t->type != T_Q4_K || (t->K % 2048) != 0 || (reinterpret_cast<uintptr_t>(t->dev) % 16) != 0) return;
    if ((reinterpret_cast<uintptr_t>(w.attn_norm.dev) % 16) != 0 || (reinterpret_cast<uintptr_t>(w.ffn_norm.dev) % 16) != 0) return;
    host[l] = TokenLayerW{w.wq.dev, w.wk.dev, w.wv.dev, w.wo.dev, w.gate.dev, w.up.dev, w.down.dev,
                          reinterpret_cast<const float*>(w.attn_norm.dev), reinterpret_cast<const float*>(w.ffn_norm.dev)};
  }
  TokenArgs probe = token_args(s);
  if (!llama_token_supported(probe, s->fa_splits, c.n_ctx)) return;
  if (c.n_head > emelb_ctx::kTokenCounters) return;   // one arrival counter per group of query heads
  // the widest product's block-value table: rows padded to 4, K/256 floats each
  const uint64_t need = std::max<uint64_t>((uint64_t)c.n_embd * (c.n_ff / 256), (uint64_t)c.n_embd * (c.n_head * c.head_dim / 256));
  if (need > s->c->bv_table_floats || (uint64_t)(2 * c.n_ff + 3) / 4 > s->c->grp_cnt_ints) return;
  if (!s->token_layers && !dev_alloc(s, (void**)&s->token_layers, sizeof(TokenLayerW) * (size_t)c.n_layer)) return;
  if (cudaMemcpyAsync(s->token_layers, host.data(), sizeof(TokenLayerW) * host.size(), cudaMemcpyHostToDevice, s->c->stream) != cudaSuccess ||
      cudaStreamSynchronize(s->c->stream) != cudaSuccess) {
    cudaGetLastError();
    return;
  }
  s->token_usable = true;
}

struct Enqueue {
  emelb_llama* s;
  cudaStream_t st;
  int launches = 0;
  bool ok = true;
  int batch_family = 0;  // family the planes were last quantized for by batch_matmul
  bool batch_tc_tiled = false;  // the tensor-core workspace holds the current planes in operand order

  Layer slot_view;       // the current layer's tensors when they are read from a window slot

  void check(cudaError_t e) { ok = ok && ctx_cuda_ok(s->c, e); }

  // Layer l's tensors for the launches that follow.  A streamed layer is asked of the window here: the view holds
  // until the next call, and the window orders its copies against this stream.  On a failed acquire `ok` drops and
  // the caller must launch nothing for the layer
  const Layer& layer_weights(int l) {
    if (!s->streamed) return s->layers[l];
    const uint8_t* base = nullptr;
    if (emelb_window_acquire(s->window, l, &base, nullptr) != EMELB_WINDOW_OK || !base) {
      ok = false;
      return s->layers[l];
    }
    slot_view = s->layers[l];
    for (Tensor* t : {&slot_view.attn_norm, &slot_view.wq, &slot_view.wk, &slot_view.wv, &slot_view.wo, &slot_view.ffn_norm,
                      &slot_view.gate, &slot_view.up, &slot_view.down})
      if (t->win_off >= 0) t->dev = base + t->win_off;
    return slot_view;
  }

  ActPlanesMut planes() const { return ActPlanesMut{s->c->act_qs, s->c->act_d, s->c->act_bsums}; }

  // make the context's planes hold `src` (K f32) quantized for `family`
  void ensure_planes(const float* src, int K, int family) {
    if (s->planes_src == src && s->planes_family == family) return;
    check(quantize_into_planes(family == 1 ? T_Q4_K : T_Q8_0, src, 1, 1, K, planes(), st));
    ++launches;
    s->planes_src = src;
    s->planes_family = family;
  }

  void matvec(const Tensor& w, const float* x, float* y, const float* residual, bool argmax = false) {
    ensure_planes(x, w.K, family_of(w.type));
    GemvArgs a{};
    a.W = w.dev;
    a.row_bytes = w.row_bytes;
    a.M = w.M;
    a.K = w.K;
    a.act = planes_view(planes(), w.type, w.K);
    a.col0 = 0;
    a.y = y;
    a.ldy = 1;
    a.residual = residual;
    a.sched = s->c->next_sched();
    a.status = s->c->status_word();
    a.pdl = s->c->pdl & 1;
    a.part_val = s->c->part_val;
    a.part_idx = s->c->part_idx;
    a.best_val = s->c->best_val;
    a.best_idx = s->c->best_idx;
    check(launch_gemv(w.type, a, 1, argmax, s->c->sm_count, st, &launches));
  }

  // several matrices of one type and K against the same activations: one launch when the
  // streaming kernel takes the shape, else one launch each
  void matvec_group(const Tensor* const* w, float* const* y, int n, const float* x) {
    bool same = n >= 2 && n <= 3;
    for (int i = 1; same && i < n; ++i) same = w[i]->type == w[0]->type && w[i]->K == w[0]->K && w[i]->row_bytes == w[0]->row_bytes;
    for (int i = 0; same && i < n; ++i) same = gemv_fast_path_ok(w[i]->type, w[i]->dev, w[i]->row_bytes, w[i]->K);
    if (!same) {
      for (int i = 0; i < n; ++i) matvec(*w[i], x, y[i], nullptr);
      return;
    }
    ensure_planes(x, w[0]->K, family_of(w[0]->type));
    GemvArgs a{};
    a.W = w[0]->dev;
    a.row_bytes = w[0]->row_bytes;
    a.M = w[0]->M;
    a.K = w[0]->K;
    a.act = planes_view(planes(), w[0]->type, w[0]->K);
    a.y = y[0];
    a.ldy = 1;
    a.W2 = w[1]->dev; a.M2 = w[1]->M; a.y2 = y[1];
    if (n == 3) { a.W3 = w[2]->dev; a.M3 = w[2]->M; a.y3 = y[2]; }
    a.sched = s->c->next_sched();
    a.status = s->c->status_word();
    a.pdl = s->c->pdl & 1;
    check(launch_gemv(w[0]->type, a, 1, false, s->c->sm_count, st, &launches));
  }

  void rms_norm(const float* x, const Tensor& w, int family) {
    check(launch_rms_norm(x, reinterpret_cast<const float*>(w.dev), s->cfg.rms_eps, s->cfg.n_embd, s->norm, family,
                          planes(), st));
    ++launches;
    s->planes_src = s->norm;
    s->planes_family = family;
  }

  // norm(x) -> up to three matrices of one type, or the argmax head.  When the streaming kernel takes the
  // shapes, the normalisation and quantization run inside the mat-vec launch (no rms_norm kernel).
  // rope_layer >= 0: the group is this layer's Q, K, V and the launch also applies RoPE and writes the KV rows;
  // returns whether that happened (false: the caller runs the RoPE / KV-store kernel)
  // whether the normalisation of x can run inside the launch of this group of matrices
  bool group_fusable(const float* x, const Tensor& nw, const Tensor* const* w, int n) const {
    bool fuse = (reinterpret_cast<uintptr_t>(x) % 16) == 0 &&
                (reinterpret_cast<uintptr_t>(nw.dev) % 16) == 0 && n >= 1 && n <= 3;
    for (int i = 0; fuse && i < n; ++i)
      fuse = gemv_prologue_supported(w[i]->type, w[i]->dev, w[i]->row_bytes, w[i]->K) && w[i]->type == w[0]->type &&
             w[i]->K == w[0]->K && w[i]->row_bytes == w[0]->row_bytes && w[i]->K == s->cfg.n_embd;
    return fuse;
  }

  // ---- joins fused into the kernels either side of them (peers attached).  One flag row, sequence counter and
  // block counter per join of a layer; row 0 belongs to the stand-alone join kernel.
  enum JoinId { J_NONE = 0, J_ATTN = 1, J_HIDDEN_A = 2, J_FFN = 3, J_HIDDEN_B = 4 };
  const JoinOut* join_out(int id) const { return id == J_NONE || !s->join_out_dev ? nullptr : s->join_out_dev + id; }
  const JoinIn* join_in(int id) const { return id == J_NONE || !s->join_in_dev ? nullptr : s->join_in_dev + id; }
  // whether every join of layer l can run inside its neighbours: the split-KV merge step produces the attention
  // context, and every product of the layer takes the streaming kernel with the quantization in its prologue
  bool layer_joins_fusable(int l) const {
    if (s->G <= 1 || !s->peers_attached || !s->join_out_dev || !s->fused_joins || s->c->attention_mode != 0) return false;
    const emelb_llama_config& c = s->cfg;
    const Layer& w = s->layers[l];
    const int64_t q_l = (int64_t)(c.n_head / s->G) * c.head_dim;
    if (q_l % 256 != 0 || (c.n_ff / s->G) % 256 != 0 || !flash_split_supported(flash_args(l))) return false;
    const Tensor* qkv[3] = {&w.wq, &w.wk, &w.wv};
    const Tensor* gu[2] = {&w.gate, &w.up};
    if (!group_fusable(s->hidden, w.attn_norm, qkv, 3) || !group_fusable(s->hidden, w.ffn_norm, gu, 2)) return false;
    const Tensor* ws[2] = {&w.wo, &w.down};
    for (const Tensor* t : ws)
      if (!gemv_prologue_supported(t->type, t->dev, t->row_bytes, t->K) || t->M % 4 != 0) return false;
    return true;
  }
  // y (this rank's rows) = [residual +] w x, x the joined vector whose Q8_K planes the producers of join `in` have
  // written into this rank's arena: the launch waits for that join and, with `out`, writes its rows to every rank
  void joined_matvec(const Tensor& w, const ActPlanesMut& x_planes, float* y, const float* residual, int in, int out) {
    GemvArgs a{};
    a.W = w.dev;
    a.row_bytes = w.row_bytes;
    a.M = w.M;
    a.K = w.K;
    a.act = planes_view(x_planes, w.type, w.K);
    a.y = y;
    a.ldy = 1;
    a.residual = residual;
    a.join_in = join_in(in);
    a.join_out = join_out(out);   // the descriptor's offset is this rank's interval of the hidden vector (== y)
    a.sched = s->c->next_sched();
    a.status = s->c->status_word();
    a.pdl = s->c->pdl & 1;
    check(launch_gemv(w.type, a, 1, false, s->c->sm_count, st, &launches));
  }

  bool normed_matvec_group(const float* x, const Tensor& nw, const Tensor* const* w, float* const* y, int n, bool argmax = false,
                           int rope_layer = -1, int in_join = 0) {
    const bool fuse = group_fusable(x, nw, w, n);
    if (!fuse && n == 3 && rope_layer >= 0 && !argmax && in_join == 0 && s->G == 1) {
      // Q / K / V of different weight types (a Q6_K value projection beside Q4_K ones): one launch per run of equal
      // types, each with the normalisation in its prologue and its part of the RoPE / KV-store epilogue
      const emelb_llama_config& cfg = s->cfg;
      int first[4] = {0, 0, 0, 0}, runs = 0;
      for (int i = 0; i < 3; ++i)
        if (i == 0 || w[i]->type != w[i - 1]->type) first[runs++] = i;
      first[runs] = 3;
      bool all = !cfg.rope_neox && cfg.head_dim % 2 == 0;
      for (int r = 0; all && r < runs; ++r) all = group_fusable(x, nw, w + first[r], first[r + 1] - first[r]);
      for (int i = 0; all && i < 3; ++i) all = w[i]->M % cfg.head_dim == 0;
      if (all) {
        for (int r = 0; r < runs; ++r) fused_group_launch(x, nw, w + first[r], y + first[r], first[r + 1] - first[r], false, rope_layer, 0, first[r]);
        s->planes_src = nullptr;
        return true;
      }
    }
    if (!fuse) {
      rms_norm(x, nw, family_of(w[0]->type));
      if (n == 1) matvec(*w[0], s->norm, y ? y[0] : nullptr, nullptr, argmax);
      else matvec_group(w, y, n, s->norm);
      return false;
    }
    const emelb_llama_config& cfg = s->cfg;
    const bool rope = rope_layer >= 0 && n == 3 && !cfg.rope_neox && cfg.head_dim % 2 == 0 && w[0]->M % cfg.head_dim == 0;
    fused_group_launch(x, nw, w, y, n, argmax, rope ? rope_layer : -1, in_join, 0);
    s->planes_src = nullptr;
    return rope;
  }

  // one launch of the streaming kernel for 1-3 matrices of one type with the rms_norm prologue; rope_layer >= 0 adds the
  // RoPE / KV-store epilogue, seg0 saying which of Q / K / V the first matrix is
  void fused_group_launch(const float* x, const Tensor& nw, const Tensor* const* w, float* const* y, int n, bool argmax,
                          int rope_layer, int in_join, int seg0) {
    const emelb_llama_config& cfg = s->cfg;
    const bool rope = rope_layer >= 0;
    GemvArgs a{};
    a.W = w[0]->dev;
    a.row_bytes = w[0]->row_bytes;
    a.M = w[0]->M;
    a.K = w[0]->K;
    a.act = planes_view(planes(), w[0]->type, w[0]->K);   // unused by the fused prologue
    a.y = y ? y[0] : nullptr;
    a.ldy = 1;
    if (n >= 2) { a.W2 = w[1]->dev; a.M2 = w[1]->M; a.y2 = y[1]; }
    if (n == 3) { a.W3 = w[2]->dev; a.M3 = w[2]->M; a.y3 = y[2]; }
    a.pro_x = x;
    a.pro_w = reinterpret_cast<const float*>(nw.dev);
    a.pro_eps = s->cfg.rms_eps;
    a.join_in = join_in(in_join);
    if (rope) {
      const int64_t layer_off = cache_off(s, rope_layer, s->cur_seq);
      a.rope_cos = s->rope_cos;
      a.rope_sin = s->rope_sin;
      a.rope_pos = s->state + 1;
      a.rope_head_dim = cfg.head_dim;
      a.rope_rot_dim = cfg.rope_dim < cfg.head_dim ? cfg.rope_dim : cfg.head_dim;
      a.rope_seg0 = seg0;
      a.rope_kcache = s->kcache + layer_off;
      a.rope_vcache = s->vcache + layer_off;
      a.rope_cache_head_stride = s->capacity * cfg.head_dim;
    }
    a.sched = s->c->next_sched();
    a.status = s->c->status_word();
    a.pdl = s->c->pdl & 1;
    a.part_val = s->c->part_val;
    a.part_idx = s->c->part_idx;
    a.best_val = s->c->best_val;
    a.best_idx = s->c->best_idx;
    check(launch_gemv(w[0]->type, a, 1, argmax, s->c->sm_count, st, &launches));
  }

  // attention of one layer; when the split-KV kernels run unsharded, their merge step also leaves the
  // context quantized for the output projection (family of wo's type)
  FlashArgs flash_args(int layer) const {
    const emelb_llama_config& c = s->cfg;
    const int64_t layer_off = cache_off(s, layer, s->cur_seq);
    FlashArgs a{};
    a.q = s->q;
    a.k = s->kcache + layer_off;
    a.v = s->vcache + layer_off;
    a.dst = s->attn + (size_t)s->rank * (c.n_head / s->G) * c.head_dim;
    a.k_nb1 = a.v_nb1 = 2 * c.head_dim;
    a.k_nb2 = a.v_nb2 = 2 * s->capacity * c.head_dim;
    a.head_dim = c.head_dim;
    a.heads = c.n_head / s->G;
    a.kv_heads = c.n_head_kv / s->G;
    a.tokens = c.n_ctx;            // upper bound; the live count is read on the device
    a.tokens_dev = s->state + 2;
    a.scale = 1.0f / std::sqrt((float)c.head_dim);
    a.splits = s->fa_splits;
    a.part_acc = s->c->fa_part_acc;
    a.part_ml = s->c->fa_part_ml;
    return a;
  }
  void attention(int layer, int out_family, int out_join = 0) {
    const emelb_llama_config& c = s->cfg;
    FlashArgs a = flash_args(layer);
    a.join_out = join_out(out_join);
    if (s->c->attention_mode == 0 && flash_split_supported(a)) {
      const bool fuse = s->G == 1 && flash_merge_can_quantize(a);
      check(launch_flash_decode(a, s->c->sm_count, st, &launches, fuse ? out_family : 0, planes()));
      if (fuse) {
        s->planes_src = s->attn;
        s->planes_family = out_family;
      }
    } else {
      check(launch_flash_reference_order(a, s->c->fa_scores, c.n_ctx, s->c->attention_mode == 1 ? 1 : 2, st, &launches));
    }
  }

  // join the ranks' row intervals of a full-length vector inside the arena (no-op unsharded)
  void gather_bytes(void* full, size_t bytes_per_rank) {
    if (s->G <= 1) return;
    if (!s->peers_attached) {
      check(comm_all_gather_bytes(s->c, full, bytes_per_rank, st));
      return;
    }
    PeerGatherArgs a{};
    a.local_base = s->arena;
    for (int g = 0; g < s->G; ++g) a.peer_base[g] = s->peer_base[g];
    a.offset_bytes = (size_t)(static_cast<char*>(full) - s->arena) + (size_t)s->rank * bytes_per_rank;
    a.bytes_per_rank = bytes_per_rank;
    a.flags_offset = s->flags_off;
    a.seq = reinterpret_cast<unsigned int*>(s->arena + s->seq_off);
    a.rank = s->rank;
    a.world = s->G;
    a.status = s->c->status_word();
    a.wait_ns = s->c->peer_wait_ns;
    check(launch_peer_gather(a, st));
    ++launches;
  }
  void gather(float* full, size_t count_per_rank) { gather_bytes(full, count_per_rank * sizeof(float)); }

  // y {w.M, B} = w x quantized(x {w.K, B}); the Q4_K products of 32 and more tokens run on the tensor cores
  // residual_inplace: y += w x where the product's kernel can add on store (y is then both addend and result);
  // returns whether it did -- otherwise y holds the bare product and the caller adds
  bool batch_matmul(const Tensor& w, const float* x, float* y, int B, bool same_input = false, bool residual_inplace = false) {
    // same_input: the planes still hold x quantized for this family (the previous product read the same x)
    bool requantized = false;
    if (!same_input || batch_family != family_of(w.type)) {
      check(quantize_into_planes(w.type, x, B, B, w.K, planes(), st));
      ++launches;
      batch_family = family_of(w.type);
      requantized = true;
    }
    if (requantized) batch_tc_tiled = false;
    GemvArgs a{};
    a.W = w.dev;
    a.row_bytes = w.row_bytes;
    a.M = w.M;
    a.K = w.K;
    a.act = planes_view(planes(), w.type, w.K);
    a.col0 = 0;
    a.y = y;
    a.ldy = B;
    a.tc_ws = s->c->tc_ws;
    a.tc_ws_bytes = s->c->tc_ws_bytes;
    // the tensor-core product keeps its own operand-ordered copy of the planes: still good for the next
    // Q4_K product of the same input
    const bool tc = gemv_takes_tensor_core(w.type, a, B);
    a.tc_ws_reuse = tc && batch_tc_tiled ? 1 : 0;
    if (tc) batch_tc_tiled = true;
    a.sched = s->c->next_sched();
    a.status = s->c->status_word();
    a.part_val = s->c->part_val;
    a.part_idx = s->c->part_idx;
    a.best_val = s->c->best_val;
    a.best_idx = s->c->best_idx;
    bool added = false;
    if (residual_inplace) {
      a.residual = y;
      added = gemm_q4k_mma_supported(w.type, a, B);
      if (!added) a.residual = nullptr;
    }
    check(launch_gemv(w.type, a, B, false, s->c->sm_count, st, &launches));
    return added;
  }

  // up to three matrices of one type and K against the same batch (Q, K, V or gate, up): one launch where the
  // 16-column tensor-core kernel takes the group, else one product each
  void batch_matmul_group(const Tensor* const* w, float* const* y, int n, const float* x, int B, bool quantized = false) {
    bool same = n >= 2 && n <= 3;
    for (int i = 1; same && i < n; ++i) same = w[i]->type == w[0]->type && w[i]->K == w[0]->K && w[i]->row_bytes == w[0]->row_bytes;
    GemvArgs a{};
    if (same) {
      a.W = w[0]->dev;
      a.row_bytes = w[0]->row_bytes;
      a.M = w[0]->M;
      a.K = w[0]->K;
      a.act = planes_view(planes(), w[0]->type, w[0]->K);
      a.y = y[0];
      a.ldy = B;
      a.W2 = w[1]->dev; a.M2 = w[1]->M; a.y2 = y[1];
      if (n == 3) { a.W3 = w[2]->dev; a.M3 = w[2]->M; a.y3 = y[2]; }
      same = gemm_q4k_mma_supported(w[0]->type, a, B);
    }
    if (!same) {
      for (int i = 0; i < n; ++i) batch_matmul(*w[i], x, y[i], B, quantized || i > 0);
      return;
    }
    if (!quantized) {
      check(quantize_into_planes(w[0]->type, x, B, B, w[0]->K, planes(), st));
      ++launches;
      batch_family = family_of(w[0]->type);
      batch_tc_tiled = false;
    }
    a.sched = s->c->next_sched();
    a.status = s->c->status_word();
    check(launch_gemv(w[0]->type, a, B, false, s->c->sm_count, st, &launches));
  }

  // B prompt tokens (ids in s->batch_tokens) at positions pos0 .. pos0 + B - 1 through every layer: fills the
  // KV cache rows of those positions.  Same arithmetic per token as token_step except the attention, which
  // is the f32 online-softmax kernel for token batches (attention mode 0 only).
  // join the ranks' row intervals of a batch tensor {rows, B}: rows are feature-major, so a rank's interval
  // is one contiguous block (NCCL all-gather in place; no-op unsharded)
  void batch_gather(float* full, size_t rows_per_rank, int B) {
    if (s->G <= 1) return;
    check(comm_all_gather_bytes(s->c, full, rows_per_rank * (size_t)B * sizeof(float), st));
    ++launches;
  }

  void prefill_chunk(int B, int pos0) {
    const emelb_llama_config& c = s->cfg;
    const int G = s->G, r = s->rank;
    const int heads_l = c.n_head / G, kv_l = c.n_head_kv / G;
    const size_t q_l = (size_t)heads_l * c.head_dim, embd_l = (size_t)c.n_embd / G, ff_l = (size_t)c.n_ff / G, b = (size_t)B;
    const int rot = c.rope_dim < c.head_dim ? c.rope_dim : c.head_dim;
    // this rank's row intervals inside the full-length batch tensors
    float* attn_mine = s->b_attn + r * q_l * b;
    float* y_mine = s->b_y + r * embd_l * b;
    float* ffn_mine = s->b_ffn + r * ff_l * b;
    s->planes_src = nullptr;
    check(launch_embed_rows(s->tok_embd.type, s->tok_embd.dev, s->tok_embd.row_bytes, s->batch_tokens, B, s->b_hidden, c.n_embd, st));
    ++launches;
    for (int l = 0; l < c.n_layer; ++l) {
      const Layer& w = layer_weights(l);
      if (!ok) break;
      const int64_t layer_off = cache_off(s, l, s->cur_seq);
      check(launch_rms_norm_batch(s->b_hidden, reinterpret_cast<const float*>(w.attn_norm.dev), c.rms_eps, c.n_embd, B, s->b_norm, s->b_partial, st));
      ++launches;
      batch_matmul(w.wq, s->b_norm, s->b_q, B);
      batch_matmul(w.wk, s->b_norm, s->b_k, B, true);
      batch_matmul(w.wv, s->b_norm, s->b_v, B, true);
      check(launch_rope_store_batch(s->b_q, s->b_k, s->b_v, s->rope_cos, s->rope_sin, pos0, B, heads_l, kv_l, c.head_dim,
                                    rot, c.rope_neox, s->kcache + layer_off, s->vcache + layer_off, s->capacity * c.head_dim, st));
      ++launches;
      PrefillAttnArgs pa{s->b_q, attn_mine, s->kcache + layer_off, s->vcache + layer_off, s->capacity * c.head_dim,
                         c.head_dim, heads_l, kv_l, B, pos0, 1.0f / std::sqrt((float)c.head_dim)};
      check(launch_prefill_attention(pa, st));
      ++launches;
      batch_gather(s->b_attn, q_l, B);
      batch_matmul(w.wo, s->b_attn, y_mine, B);
      batch_gather(s->b_y, embd_l, B);
      check(launch_add_inplace(s->b_hidden, s->b_y, (int64_t)c.n_embd * B, st));
      check(launch_rms_norm_batch(s->b_hidden, reinterpret_cast<const float*>(w.ffn_norm.dev), c.rms_eps, c.n_embd, B, s->b_norm, s->b_partial, st));
      batch_matmul(w.gate, s->b_norm, s->b_gate, B);
      batch_matmul(w.up, s->b_norm, s->b_up, B, true);
      check(launch_swiglu(s->b_gate, s->b_up, (int)(ff_l * b), ffn_mine, 0, planes(), st));
      batch_gather(s->b_ffn, ff_l, B);
      batch_matmul(w.down, s->b_ffn, y_mine, B);
      batch_gather(s->b_y, embd_l, B);
      check(launch_add_inplace(s->b_hidden, s->b_y, (int64_t)c.n_embd * B, st));
      launches += 4;
    }
  }

  // One decode step of sequences 0 .. B-1 together: column j of every activation tensor {features, B} is sequence
  // j's token (ids, positions and token counts in s->bstate).  Per column the arithmetic is token_step's: the
  // same products, the same rotation, the split-KV attention with the session's split count, so a sequence
  // decodes to the tokens it decodes to alone.  Ends with the per-column argmax (and the logits left in
  // s->b_logits, {n_vocab, B}).
  void batch_step(int B) {
    const emelb_llama_config& c = s->cfg;
    const int G = s->G, r = s->rank;
    const int heads_l = c.n_head / G, kv_l = c.n_head_kv / G;
    const size_t q_l = (size_t)heads_l * c.head_dim, embd_l = (size_t)c.n_embd / G, ff_l = (size_t)c.n_ff / G, b = (size_t)B;
    const size_t vocab_l = (size_t)c.n_vocab / G;
    const int rot = c.rope_dim < c.head_dim ? c.rope_dim : c.head_dim;
    float* attn_mine = s->b_attn + r * q_l * b;
    float* y_mine = s->b_y + r * embd_l * b;
    float* ffn_mine = s->b_ffn + r * ff_l * b;
    const int* tok = s->bstate;
    const int* pos = s->bstate + kMaxSeqs;
    const int* kvn = s->bstate + 2 * kMaxSeqs;
    s->planes_src = nullptr;
    // rms_norm of the batch for a product of weight type `type`: with K-quant weights one launch leaves the Q8_K
    // planes (true: the product need not quantize), else the f32 result goes to b_norm
    auto norm = [&](const Tensor& nw, int type) {
      if (family_of(type) == 1 && B <= 64) {
        check(launch_rms_norm_quant_cols(s->b_hidden, reinterpret_cast<const float*>(nw.dev), c.rms_eps, c.n_embd, B, planes(), st));
        ++launches;
        batch_family = 1;
        batch_tc_tiled = false;
        return true;
      }
      check(launch_rms_norm_batch(s->b_hidden, reinterpret_cast<const float*>(nw.dev), c.rms_eps, c.n_embd, B, s->b_norm, s->b_partial, st));
      launches += 2;
      return false;
    };
    // b_hidden += w x: unsharded, the product's kernel adds on store where it can; else the product goes to this
    // rank's rows of b_y, the rows are joined, and one kernel adds
    auto residual_product = [&](const Tensor& w, const float* x, float* y_rows, int cols, bool quantized) {
      if (G == 1) {
        GemvArgs probe{};
        probe.W = w.dev;
        probe.row_bytes = w.row_bytes;
        probe.M = w.M;
        probe.K = w.K;
        probe.act = planes_view(planes(), w.type, w.K);
        probe.residual = s->b_hidden;
        if (gemm_q4k_mma_supported(w.type, probe, cols)) {
          batch_matmul(w, x, s->b_hidden, cols, quantized, true);
          return;
        }
      }
      batch_matmul(w, x, y_rows, cols, quantized);
      batch_gather(s->b_y, embd_l, cols);
      check(launch_add_inplace(s->b_hidden, s->b_y, (int64_t)c.n_embd * cols, st));
      ++launches;
    };
    check(launch_embed_rows(s->tok_embd.type, s->tok_embd.dev, s->tok_embd.row_bytes, tok, B, s->b_hidden, c.n_embd, st));
    ++launches;
    for (int l = 0; l < c.n_layer; ++l) {
      const Layer& w = layer_weights(l);
      if (!ok) break;
      const int64_t layer_off = cache_off(s, l, 0);
      {
        const bool same_type = w.wk.type == w.wq.type && w.wv.type == w.wq.type;
        const bool quantized = same_type ? norm(w.attn_norm, w.wq.type) : (norm(w.attn_norm, T_F32), false);
        const Tensor* ws[3] = {&w.wq, &w.wk, &w.wv};
        float* ys[3] = {s->b_q, s->b_k, s->b_v};
        batch_matmul_group(ws, ys, 3, s->b_norm, B, quantized);
      }
      check(launch_rope_store_seqs(s->b_q, s->b_k, s->b_v, s->rope_cos, s->rope_sin, pos, B, heads_l, kv_l, c.head_dim, rot,
                                   c.rope_neox, s->b_qs, s->kcache + layer_off, s->vcache + layer_off,
                                   (int64_t)kv_l * s->capacity * c.head_dim, s->capacity * c.head_dim, st));
      ++launches;
      // every (sequence, head) is one head of a wider attention problem over the sequences' cache planes
      FlashArgs a = flash_args(l);
      a.q = s->b_qs;
      a.k = s->kcache + layer_off;
      a.v = s->vcache + layer_off;
      a.dst = attn_mine;
      a.heads = heads_l * B;
      a.kv_heads = kv_l * B;
      a.tokens_dev = kvn;
      a.kv_heads_per_seq = kv_l;
      a.dst_seqs = B;
      a.part_acc = s->b_part_acc;
      a.part_ml = s->b_part_ml;
      // unsharded with K-quant weights: the merge step leaves each sequence's context quantized for Wo, and the
      // products add the residual on store
      const bool attn_q = G == 1 && family_of(w.wo.type) == 1 && q_l % 256 == 0;
      check(launch_flash_decode(a, s->c->sm_count, st, &launches, attn_q ? 1 : 0, planes()));
      if (attn_q) {
        batch_family = 1;
        batch_tc_tiled = false;
      }
      batch_gather(s->b_attn, q_l, B);
      residual_product(w.wo, s->b_attn, y_mine, B, attn_q);
      {
        const bool quantized = w.up.type == w.gate.type ? norm(w.ffn_norm, w.gate.type) : (norm(w.ffn_norm, T_F32), false);
        const Tensor* ws[2] = {&w.gate, &w.up};
        float* ys[2] = {s->b_gate, s->b_up};
        batch_matmul_group(ws, ys, 2, s->b_norm, B, quantized);
      }
      const bool ffn_q = G == 1 && family_of(w.down.type) == 1 && B <= 64;
      if (ffn_q) {
        check(launch_swiglu_quant_cols(s->b_gate, s->b_up, c.n_ff, B, planes(), st));
        batch_family = 1;
        batch_tc_tiled = false;
      } else {
        check(launch_swiglu(s->b_gate, s->b_up, (int)(ff_l * b), ffn_mine, 0, planes(), st));
      }
      ++launches;
      batch_gather(s->b_ffn, ff_l, B);
      residual_product(w.down, s->b_ffn, y_mine, B, ffn_q);
    }
    const bool quantized = norm(s->out_norm, s->output.type);
    batch_matmul(s->output, s->b_norm, s->b_logits + r * vocab_l * b, B, quantized);
    batch_gather(s->b_logits, vocab_l, B);
    check(launch_argmax_columns(s->b_logits, c.n_vocab, B, s->b_amax_val, s->b_amax_idx, s->b_idx, st));
    launches += 2;
  }

  void token_step(Mode mode) {
    const emelb_llama_config& c = s->cfg;
    // which launches of the step carry the programmatic-serialization attribute (bit mask: 1 mat-vecs,
    // 2 RoPE/KV store, 4 attention, 8 SwiGLU, 16 the rest); the flag is read by EMELB_LAUNCH
    struct PdlScope {
      explicit PdlScope(bool on) { g_pdl_launch = on; }
      ~PdlScope() { g_pdl_launch = false; }
    };
    const int pm = s->c->pdl;
    PdlScope pdl_rest((pm & 16) != 0);
    const int G = s->G, r = s->rank;
    const int heads_l = c.n_head / G, kv_l = c.n_head_kv / G;
    const size_t q_l = (size_t)heads_l * c.head_dim, embd_l = (size_t)c.n_embd / G, ff_l = (size_t)c.n_ff / G;
    float* hidden_mine = s->hidden + r * embd_l;
    s->planes_src = nullptr;
    check(launch_embed_row(s->tok_embd.type, s->tok_embd.dev, s->tok_embd.row_bytes, s->state, s->hidden, c.n_embd, st));
    ++launches;
    const bool one_kernel = s->token_usable && s->step_mode == 1 && s->c->attention_mode == 0 && G == 1 && s->n_seq == 1;
    if (one_kernel) {
      // every layer inside one persistent kernel (token_kernel.cu)
      check(launch_llama_token(token_args(s), s->c->sm_count, &s->token_launch, st));
      ++launches;
    }
    bool hidden_joined_in_next = false;   // the previous layer left the join of the hidden vector to this layer's first launch
    for (int l = 0; l < c.n_layer && !one_kernel; ++l) {
      const Layer& w = layer_weights(l);
      if (!ok) break;
      bool roped = false;
      {
        const Tensor* ws[3] = {&w.wq, &w.wk, &w.wv};
        float* ys[3] = {s->q, s->k, s->v};
        roped = normed_matvec_group(s->hidden, w.attn_norm, ws, ys, 3, false, l, hidden_joined_in_next ? J_HIDDEN_B : J_NONE);
      }
      if (!roped) {
        const int64_t layer_off = cache_off(s, l, s->cur_seq);
        g_pdl_launch = (pm & 2) != 0;
        check(launch_rope_store(s->q, s->k, s->v, s->rope_cos, s->rope_sin, s->state + 1, heads_l, kv_l, c.head_dim,
                                c.rope_dim < c.head_dim ? c.rope_dim : c.head_dim, c.rope_neox, s->kcache + layer_off,
                                s->vcache + layer_off, s->capacity * c.head_dim, st));
        ++launches;
      }
      // joins of this layer inside its kernels (peers attached and every product qualifies), else one join kernel
      // (or NCCL call) each; the hidden vector after the down projection is joined inside the next layer's first
      // launch only when that layer qualifies too
      const bool fj = layer_joins_fusable(l);
      const bool fj_next = fj && l + 1 < c.n_layer && layer_joins_fusable(l + 1);
      g_pdl_launch = (pm & 4) != 0;
      attention(l, family_of(w.wo.type), fj ? J_ATTN : J_NONE);
      g_pdl_launch = (pm & 16) != 0;
      if (fj) {
        joined_matvec(w.wo, s->attn_planes, hidden_mine, hidden_mine, J_ATTN, J_HIDDEN_A);   // hidden += Wo * attn (this rank's rows)
      } else {
        gather(s->attn, q_l);
        matvec(w.wo, s->attn, hidden_mine, hidden_mine);
        gather(s->hidden, embd_l);
      }
      {
        const Tensor* ws[2] = {&w.gate, &w.up};
        float* ys[2] = {s->gate, s->up};
        normed_matvec_group(s->hidden, w.ffn_norm, ws, ys, 2, false, -1, fj ? J_HIDDEN_A : J_NONE);
      }
      g_pdl_launch = (pm & 8) != 0;
      if (G == 1) {
        check(launch_swiglu(s->gate, s->up, c.n_ff, nullptr, family_of(w.down.type), planes(), st));  // only the quantized product is consumed
        s->planes_src = s->ffn;
        s->planes_family = family_of(w.down.type);
      } else if (fj) {
        check(launch_swiglu_join(s->gate, s->up, (int)ff_l, join_out(J_FFN), st));
        s->planes_src = nullptr;
      } else {
        // the product is quantized after the join, over the full vector
        check(launch_swiglu(s->gate, s->up, (int)ff_l, s->ffn + r * ff_l, 0, planes(), st));
        s->planes_src = nullptr;
      }
      ++launches;
      g_pdl_launch = (pm & 16) != 0;
      if (fj) {
        joined_matvec(w.down, s->ffn_planes, hidden_mine, hidden_mine, J_FFN, fj_next ? J_HIDDEN_B : J_NONE);   // hidden += Wdown * ffn
        if (!fj_next) gather(s->hidden, embd_l);
      } else {
        gather(s->ffn, ff_l);
        matvec(w.down, s->ffn, hidden_mine, hidden_mine);
        gather(s->hidden, embd_l);
      }
      hidden_joined_in_next = fj_next;
    }
    if (mode == MODE_PREFILL) return;
    const size_t vocab_l = (size_t)c.n_vocab / G;
    const Tensor* head[1] = {&s->output};
    if (mode == MODE_ARGMAX) {
      normed_matvec_group(s->hidden, s->out_norm, head, nullptr, 1, true);
      if (G > 1) {
        // candidates {value, global row} of every rank, then the same lowest-row tie rule
        check(launch_argmax_pair_store(s->c->best_val, s->c->best_idx, (int)(r * vocab_l), s->pair_buf + 4 * r, st));
        gather_bytes(s->pair_buf, 4 * sizeof(int));
        check(launch_argmax_pair_finish(s->pair_buf, G, s->c->best_val, s->c->best_idx, st));
        launches += 2;
      }
      check(launch_step_advance(s->state, s->c->best_idx, s->tokens_dev, st));
      ++launches;
    } else {
      float* ys[1] = {s->logits + r * vocab_l};
      normed_matvec_group(s->hidden, s->out_norm, head, ys, 1);
      gather(s->logits, vocab_l);
    }
  }
};

// capture (once per mode and attention mode) and return the replayable step.  The eager pass that precedes a
// capture is a real step: it runs for (token, position), the step the caller is about to replay, so the KV row
// it writes is the one the replay writes again (a stale position would overwrite a live row of the cache)
cudaGraphExec_t step_graph(emelb_llama* s, Mode mode, int token, int position) {
  if (s->graphs[mode] && s->graph_attention_mode[mode] == s->c->attention_mode) return s->graphs[mode];
  if (s->graphs[mode]) {
    cudaStreamSynchronize(s->c->stream);
    cudaGraphExecDestroy(s->graphs[mode]);
    s->graphs[mode] = nullptr;
  }
  prepare_token_kernel(s);
  // one eager pass first: sets per-kernel attributes outside the capture
  if (!ctx_cuda_ok(s->c, launch_step_begin(s->state, token, position, s->c->stream))) return nullptr;
  Enqueue warm{s, s->c->stream};
  warm.token_step(mode);
  if (!warm.ok || !ctx_cuda_ok(s->c, cudaStreamSynchronize(s->c->stream))) return nullptr;
  if (!ctx_cuda_ok(s->c, cudaStreamBeginCapture(s->c->stream, cudaStreamCaptureModeThreadLocal))) return nullptr;
  Enqueue e{s, s->c->stream};
  e.token_step(mode);
  cudaGraph_t g = nullptr;
  const bool ended = ctx_cuda_ok(s->c, cudaStreamEndCapture(s->c->stream, &g));
  if (!ended || !e.ok || !g) {
    if (g) cudaGraphDestroy(g);
    return nullptr;
  }
  cudaGraphExec_t ex = nullptr;
  const bool inst = ctx_cuda_ok(s->c, cudaGraphInstantiate(&ex, g, 0));
  cudaGraphDestroy(g);
  if (!inst) return nullptr;
  s->graphs[mode] = ex;
  s->graph_attention_mode[mode] = s->c->attention_mode;
  s->launches_mode[mode] = e.launches;
  if (mode == MODE_ARGMAX) s->launches_per_token = e.launches;
  return ex;
}

// make mode's step launchable for the device-side state: the replayable graph, or nothing when layers are streamed
// (a window acquire orders copies against the stream with events, which a replayed graph could not re-issue)
bool step_ready(emelb_llama* s, Mode mode, int token, int position) {
  if (s->streamed) return true;
  return step_graph(s, mode, token, position) != nullptr;
}

// enqueue one step of `mode`
bool step_launch(emelb_llama* s, Mode mode) {
  emelb_ctx* c = s->c;
  if (!s->streamed) {
    c->diag.kernel_launches += s->launches_mode[mode];
    return ctx_cuda_ok(c, cudaGraphLaunch(s->graphs[mode], c->stream));
  }
  Enqueue e{s, c->stream};
  e.token_step(mode);
  c->diag.kernel_launches += e.launches;
  s->launches_mode[mode] = e.launches;
  if (mode == MODE_ARGMAX) s->launches_per_token = e.launches;
  return e.ok;
}

bool valid_step(const emelb_llama* s, int token, int position) {
  return token >= 0 && token < s->cfg.n_vocab && position >= 0 && position < s->cfg.n_ctx;
}

}  // namespace

extern "C" {

uint32_t emelb_llama_check_config(const emelb_llama_config* cfg) {
  if (!cfg) return EMELB_INVALID_REQUEST;
  const emelb_llama_config& g = *cfg;
  const bool sane = g.n_layer > 0 && g.n_embd > 0 && g.n_embd % 256 == 0 && g.n_head > 0 && g.n_head_kv > 0 &&
                    g.n_head % g.n_head_kv == 0 && g.head_dim > 1 && g.n_ff > 0 && g.n_ff % 256 == 0 && g.n_vocab > 0 &&
                    g.n_ctx > 0 && g.rope_dim > 1 && g.rope_dim % 2 == 0 && g.shard_count >= 1 && g.shard_rank >= 0 &&
                    g.shard_rank < g.shard_count;
  if (!sane) return EMELB_INVALID_REQUEST;
  const int G = g.shard_count;
  if (G > 1) {
    // row intervals must be whole heads / whole rows on every rank ...
    if (G > kMaxPeers || g.n_head_kv % G != 0 || g.n_embd % G != 0 || g.n_ff % G != 0 || g.n_vocab % G != 0) return EMELB_INVALID_REQUEST;
    // ... and every interval that is joined across ranks is moved in 16-byte units: the f32 intervals of the
    // attention context, the hidden vector, the gate / up / SwiGLU vectors and the logits
    const int64_t q_l = (int64_t)g.n_head * g.head_dim / G;
    if (q_l % 4 != 0 || (g.n_embd / G) % 4 != 0 || (g.n_ff / G) % 4 != 0 || (g.n_vocab / G) % 4 != 0) return EMELB_INVALID_REQUEST;
  }
  return EMELB_OK;
}

uint32_t emelb_llama_create(emelb_ctx* c, const emelb_llama_config* cfg, emelb_llama** out) {
  if (!c || !cfg || !out) return EMELB_INVALID_REQUEST;
  *out = nullptr;
  const emelb_llama_config& g = *cfg;
  if (emelb_llama_check_config(cfg) != EMELB_OK) return EMELB_INVALID_REQUEST;
  if ((int64_t)g.n_head * g.head_dim > (int64_t)c->act_capacity || (int64_t)g.n_ff > (int64_t)c->act_capacity) return EMELB_INVALID_REQUEST;
  const int G = g.shard_count;
  // the context's communicator must match the shard layout
  if (G > 1 && (!c->comm || c->comm_world != G || c->comm_rank != g.shard_rank)) return EMELB_INVALID_REQUEST;
  cudaSetDevice(c->device);
  emelb_llama* s = new (std::nothrow) emelb_llama();
  if (!s) return EMELB_INTERNAL_ERROR;
  s->c = c;
  s->cfg = g;
  s->G = G;
  s->rank = g.shard_rank;
  s->layers.resize(g.n_layer);
  const int kvb = g.kv_block > 0 ? g.kv_block : 16;
  s->capacity = ((int64_t)g.n_ctx + kvb - 1) / kvb * kvb;
  const size_t qd = (size_t)g.n_head * g.head_dim, kvd = (size_t)g.n_head_kv * g.head_dim;
  const size_t cache_halves = (size_t)g.n_layer * (g.n_head_kv / G) * s->capacity * g.head_dim;  // this rank's KV heads
  const int pairs = (g.rope_dim < g.head_dim ? g.rope_dim : g.head_dim) / 2;
  bool ok = true;
  if (G > 1) {
    // [hidden | attn | ffn | logits | pairs | flags | seq], each part 256-byte aligned, zero-filled.  flags: five
    // rows of kMaxPeers u32 (the join kernel's, then one per fused join of a layer); seq: their sequence counters,
    // then at byte 64 their finished-block counters
    auto up = [](size_t b) { return (b + 255) & ~size_t(255); };
    const size_t o_hidden = 0, o_attn = o_hidden + up(4 * (size_t)g.n_embd), o_ffn = o_attn + up(4 * qd),
                 o_logits = o_ffn + up(4 * (size_t)g.n_ff), o_pairs = o_logits + up(4 * (size_t)g.n_vocab),
                 o_flags = o_pairs + up(16 * (size_t)kMaxPeers), o_seq = o_flags + up(5 * 4 * (size_t)kMaxPeers);
    // Q8_K planes {qs, bsums, d} of the two vectors whose producers quantize before the join
    const size_t o_aqs = o_seq + 256, o_abs = o_aqs + up(qd), o_ad = o_abs + up(qd / 8), o_fqs = o_ad + up(qd / 64),
                 o_fbs = o_fqs + up((size_t)g.n_ff), o_fd = o_fbs + up((size_t)g.n_ff / 8);
    s->arena_bytes = o_fd + up((size_t)g.n_ff / 64);
    ok = ok && dev_alloc(s, (void**)&s->arena, s->arena_bytes);
    if (ok) {
      ok = cudaMemsetAsync(s->arena, 0, s->arena_bytes, c->stream) == cudaSuccess;
      s->hidden = reinterpret_cast<float*>(s->arena + o_hidden);
      s->attn = reinterpret_cast<float*>(s->arena + o_attn);
      s->ffn = reinterpret_cast<float*>(s->arena + o_ffn);
      s->logits = reinterpret_cast<float*>(s->arena + o_logits);
      s->pair_buf = reinterpret_cast<int*>(s->arena + o_pairs);
      s->flags_off = o_flags;
      s->seq_off = o_seq;
      s->attn_planes = ActPlanesMut{reinterpret_cast<int8_t*>(s->arena + o_aqs), reinterpret_cast<float*>(s->arena + o_ad),
                                    reinterpret_cast<int16_t*>(s->arena + o_abs)};
      s->ffn_planes = ActPlanesMut{reinterpret_cast<int8_t*>(s->arena + o_fqs), reinterpret_cast<float*>(s->arena + o_fd),
                                   reinterpret_cast<int16_t*>(s->arena + o_fbs)};
      s->peer_base[g.shard_rank] = s->arena;
    }
  }
  if (G == 1) ok = ok && dev_alloc(s, (void**)&s->hidden, 4 * (size_t)g.n_embd);
  ok = ok && dev_alloc(s, (void**)&s->norm, 4 * (size_t)g.n_embd);
  ok = ok && dev_alloc(s, (void**)&s->q, 4 * qd);
  ok = ok && dev_alloc(s, (void**)&s->k, 4 * kvd);
  ok = ok && dev_alloc(s, (void**)&s->v, 4 * kvd);
  if (G == 1) ok = ok && dev_alloc(s, (void**)&s->attn, 4 * qd);
  ok = ok && dev_alloc(s, (void**)&s->gate, 4 * (size_t)g.n_ff);
  ok = ok && dev_alloc(s, (void**)&s->up, 4 * (size_t)g.n_ff);
  if (G == 1) ok = ok && dev_alloc(s, (void**)&s->ffn, 4 * (size_t)g.n_ff);
  if (G == 1) ok = ok && dev_alloc(s, (void**)&s->logits, 4 * (size_t)g.n_vocab);
  ok = ok && dev_alloc(s, (void**)&s->kcache, 2 * cache_halves);
  ok = ok && dev_alloc(s, (void**)&s->vcache, 2 * cache_halves);
  ok = ok && dev_alloc(s, (void**)&s->rope_cos, 4 * (size_t)g.n_ctx * pairs);
  ok = ok && dev_alloc(s, (void**)&s->rope_sin, 4 * (size_t)g.n_ctx * pairs);
  ok = ok && dev_alloc(s, (void**)&s->state, 4 * sizeof(int));
  if (G == 1) ok = ok && dev_alloc(s, (void**)&s->pair_buf, 4 * sizeof(int));
  ok = ok && dev_alloc(s, (void**)&s->tokens_dev, sizeof(int) * (size_t)(g.n_ctx + 8));
  ok = ok && cudaMallocHost((void**)&s->host_pinned, sizeof(int) * (size_t)(g.n_ctx + 4 + 2 * kMaxSeqs)) == cudaSuccess;
  if (ok) {
    ok = cudaMemsetAsync(s->kcache, 0, 2 * cache_halves, c->stream) == cudaSuccess &&
         cudaMemsetAsync(s->vcache, 0, 2 * cache_halves, c->stream) == cudaSuccess &&
         cudaMemsetAsync(s->state, 0, 4 * sizeof(int), c->stream) == cudaSuccess;
  }
  if (ok) {
    // cos/sin of theta_p = position * base^(-2p/rot) built with the host libm and the
    // same recurrence as apply_rope_pairing (:2918-2934), so the table holds
    // exactly the floats the reference multiplies by
    std::vector<float> hc((size_t)g.n_ctx * pairs), hs((size_t)g.n_ctx * pairs);
    const float theta_scale = ::powf(g.rope_freq_base, -2.0f / (float)(2 * pairs));
    for (int pos = 0; pos < g.n_ctx; ++pos) {
      float theta = (float)pos;
      for (int p = 0; p < pairs; ++p) {
        hc[(size_t)pos * pairs + p] = ::cosf(theta);
        hs[(size_t)pos * pairs + p] = ::sinf(theta);
        theta *= theta_scale;
      }
    }
    ok = cudaMemcpyAsync(s->rope_cos, hc.data(), hc.size() * 4, cudaMemcpyHostToDevice, c->stream) == cudaSuccess &&
         cudaMemcpyAsync(s->rope_sin, hs.data(), hs.size() * 4, cudaMemcpyHostToDevice, c->stream) == cudaSuccess &&
         cudaStreamSynchronize(c->stream) == cudaSuccess;
  }
  if (ok) {
    int max_splits = (int)(kFlashPartFloats / ((uint64_t)g.n_head * g.head_dim));
    if (max_splits > 64) max_splits = 64;
    s->fa_splits = max_splits >= 1 ? flash_pick_splits(g.n_ctx, g.n_head_kv / G, c->sm_count, max_splits) : 1;
    ok = (uint64_t)g.n_head * (uint64_t)g.n_ctx <= kFlashScoreFloats;
  }
  if (!ok) {
    cudaGetLastError();
    emelb_llama_destroy(s);
    return EMELB_INTERNAL_ERROR;
  }
  *out = s;
  return EMELB_OK;
}

uint32_t emelb_llama_destroy(emelb_llama* s) {
  if (!s) return EMELB_INVALID_REQUEST;
  cudaSetDevice(s->c->device);
  cudaStreamSynchronize(s->c->stream);
  for (auto& g : s->graphs)
    if (g) cudaGraphExecDestroy(g);
  if (s->batch_graph) cudaGraphExecDestroy(s->batch_graph);
  for (int g = 0; g < kMaxPeers; ++g)
    if (s->peer_base[g] && g != s->rank) cudaIpcCloseMemHandle(s->peer_base[g]);
  for (void* p : s->owned) cudaFree(p);
  if (s->host_pinned) cudaFreeHost(s->host_pinned);
  cudaGetLastError();
  delete s;
  return EMELB_OK;
}

uint32_t emelb_llama_bind(emelb_llama* s, int32_t layer, int32_t role, const emelb_view* t) {
  if (!s || !t || !t->data) return EMELB_INVALID_REQUEST;
  const emelb_llama_config& c = s->cfg;
  const bool model_level = role <= EMELB_T_OUTPUT;
  if (role < 0 || role > EMELB_T_FFN_DOWN || (model_level ? layer != -1 : (layer < 0 || layer >= c.n_layer)))
    return EMELB_INVALID_REQUEST;
  // a sharded session binds this rank's row interval of each matrix (M/G rows, all K columns);
  // the embedding table and the norm vectors are whole on every rank
  const int qd = c.n_head * c.head_dim, kvd = c.n_head_kv * c.head_dim, G = s->G;
  int K = 0, M = 0;
  bool vector = false;
  switch (role) {
    case EMELB_T_TOKEN_EMBD: K = c.n_embd; M = c.n_vocab; break;
    case EMELB_T_OUTPUT: K = c.n_embd; M = c.n_vocab / G; break;
    case EMELB_T_OUTPUT_NORM: case EMELB_T_ATTN_NORM: case EMELB_T_FFN_NORM: K = c.n_embd; M = 1; vector = true; break;
    case EMELB_T_ATTN_Q: K = c.n_embd; M = qd / G; break;
    case EMELB_T_ATTN_K: case EMELB_T_ATTN_V: K = c.n_embd; M = kvd / G; break;
    case EMELB_T_ATTN_OUT: K = qd; M = c.n_embd / G; break;
    case EMELB_T_FFN_GATE: case EMELB_T_FFN_UP: K = c.n_embd; M = c.n_ff / G; break;
    case EMELB_T_FFN_DOWN: K = c.n_ff; M = c.n_embd / G; break;
  }
  Tensor x;
  x.type = t->type;
  x.K = K;
  x.M = M;
  if ((int64_t)t->ne[0] != K || (int64_t)t->ne[1] != M) return EMELB_INVALID_REQUEST;
  if (vector) {
    if (t->type != EMELB_F32) return EMELB_INVALID_REQUEST;
    x.row_bytes = 4 * (int64_t)K;
  } else if (role == EMELB_T_TOKEN_EMBD && (t->type == EMELB_F32 || t->type == EMELB_F16)) {
    x.row_bytes = (t->type == EMELB_F32 ? 4 : 2) * (int64_t)K;
    if ((int64_t)t->nb[1] != x.row_bytes) return EMELB_INVALID_REQUEST;
  } else {
    const int be = block_elems(t->type);
    if (be == 0 || t->type == EMELB_Q8_K || K % be != 0) return EMELB_INVALID_REQUEST;
    const int lim = is_k_type(t->type) ? MAX_Q8_K_BLOCKS : MAX_Q8_0_BLOCKS;
    x.row_bytes = (int64_t)(K / be) * block_bytes(t->type);
    if (role != EMELB_T_TOKEN_EMBD && K / be > lim) return EMELB_INVALID_REQUEST;
    if ((int64_t)t->nb[1] != x.row_bytes || t->nb[0] != 1) return EMELB_INVALID_REQUEST;
  }
  x.dev = static_cast<const uint8_t*>(ctx_resolve_weights(s->c, t->data));
  if (!x.dev) {
    // not resident: a layer tensor may lie in the source of the session's streaming window
    uint64_t off = 0;
    if (model_level || !window_find_extent(s->window, layer, t->data, (uint64_t)x.row_bytes * (uint64_t)M, &off) || off % 16 != 0)
      return EMELB_INVALID_REQUEST;
    x.win_off = (int64_t)off;
  }
  Tensor* slot = nullptr;
  if (model_level) slot = role == EMELB_T_TOKEN_EMBD ? &s->tok_embd : (role == EMELB_T_OUTPUT_NORM ? &s->out_norm : &s->output);
  else {
    Layer& l = s->layers[layer];
    Tensor* slots[] = {&l.attn_norm, &l.wq, &l.wk, &l.wv, &l.wo, &l.ffn_norm, &l.gate, &l.up, &l.down};
    slot = slots[role - EMELB_T_ATTN_NORM];
  }
  *slot = x;
  // bindings changed: captured steps hold stale pointers
  for (int m = 0; m < MODE_COUNT; ++m) s->graph_attention_mode[m] = -1;
  s->batch_graph_mode = -1;
  s->token_layers_valid = false;
  s->streamed = streamed_tensors(s) > 0;
  return EMELB_OK;
}

uint32_t emelb_llama_set_window(emelb_llama* s, emelb_window* w) {
  if (!s) return EMELB_INVALID_REQUEST;
  // tensors bound through the previous window keep offsets into its slots: they must be bound again first
  if (streamed_tensors(s) > 0) return EMELB_INVALID_REQUEST;
  if (w) {
    // one window per unsharded session, on the session's context, with one descriptor per layer
    if (s->G != 1 || window_ctx(w) != s->c || !window_streaming(w) || window_layer_count(w) != s->cfg.n_layer) return EMELB_INVALID_REQUEST;
  }
  s->window = w;
  return EMELB_OK;
}

uint32_t emelb_llama_decode(emelb_llama* s, int32_t token, int32_t position, float* logits_out, int32_t* token_out) {
  if (!s || !valid_step(s, token, position) || !all_bound(s)) return EMELB_INVALID_REQUEST;
  emelb_ctx* c = s->c;
  cudaSetDevice(c->device);
  const Mode mode = logits_out ? MODE_LOGITS : MODE_ARGMAX;
  if (!step_ready(s, mode, token, position)) return EMELB_INTERNAL_ERROR;
  bool ok = ctx_cuda_ok(c, launch_step_begin(s->state, token, position, c->stream));
  ok = ok && step_launch(s, mode);
  c->diag.kernel_launches += 1;
  if (ok && logits_out) {
    cudaPointerAttributes at{};
    const bool dev = cudaPointerGetAttributes(&at, logits_out) == cudaSuccess && at.type == cudaMemoryTypeDevice;
    cudaGetLastError();
    ok = ctx_cuda_ok(c, cudaMemcpyAsync(logits_out, s->logits, 4 * (size_t)s->cfg.n_vocab,
                                        dev ? cudaMemcpyDeviceToDevice : cudaMemcpyDeviceToHost, c->stream));
    if (!dev) c->diag.d2h_bytes += 4 * (uint64_t)s->cfg.n_vocab;
    if (ok && token_out) {
      ok = ctx_cuda_ok(c, launch_argmax_f32(s->logits, s->cfg.n_vocab, c->best_val, c->best_idx, c->stream));
      c->diag.kernel_launches += 1;
      ok = ok && ctx_cuda_ok(c, cudaMemcpyAsync(s->host_pinned, c->best_idx, 4, cudaMemcpyDeviceToHost, c->stream));
      c->diag.d2h_bytes += 4;
    }
  } else if (ok && token_out) {
    ok = ctx_cuda_ok(c, cudaMemcpyAsync(s->host_pinned, c->best_idx, 4, cudaMemcpyDeviceToHost, c->stream));
    c->diag.d2h_bytes += 4;
  }
  ok = ok && ctx_cuda_ok(c, cudaStreamSynchronize(c->stream));
  if (ok && token_out) *token_out = s->host_pinned[0];
  return ok ? EMELB_OK : EMELB_INTERNAL_ERROR;
}

namespace {

// token-batch size of the prompt path: 0 = walk the prompt token by token.  Batches need the batch attention
// kernel (attention mode 0: the reference-order modes exist to be compared one token at a time), room for one
// batch in the context's activation planes and, in a sharded session, the context's communicator for the joins.
int prefill_batch_size(emelb_llama* s, int n) {
  const emelb_llama_config& c = s->cfg;
  if (s->prefill_batch <= 0 || s->c->attention_mode != 0 || n < 2) return 0;
  if (s->G > 1 && (!s->c->comm || s->c->comm_world != s->G)) return 0;   // batch joins go through the communicator
  PrefillAttnArgs pa{nullptr, nullptr, s->kcache, s->vcache, s->capacity * c.head_dim, c.head_dim, c.n_head / s->G,
                     c.n_head_kv / s->G, 1, 0, 1.0f};
  if (!prefill_attention_supported(pa)) return 0;
  int widest = c.n_ff > c.n_embd ? c.n_ff : c.n_embd;
  if (c.n_head * c.head_dim > widest) widest = c.n_head * c.head_dim;
  int cap = s->prefill_batch;
  const int64_t fits = (int64_t)(s->c->act_capacity / (uint64_t)widest);
  if (cap > fits) cap = (int)fits;
  if ((int64_t)c.n_ff * cap > 0x7fffffff) cap = 0x7fffffff / c.n_ff;
  return cap < 2 ? 0 : cap;
}

bool reserve_batch(emelb_llama* s, int B) {
  if (s->batch_cap > 0) return true;   // sized by the first batched prompt; later batches are cut to fit
  if (s->batch_cap < 0) return false;  // the buffers did not fit once: prompts are walked token by token
  const emelb_llama_config& c = s->cfg;
  const size_t q_dim = (size_t)c.n_head * c.head_dim, kv_dim = (size_t)c.n_head_kv * c.head_dim, b = (size_t)B;
  bool ok = dev_alloc(s, (void**)&s->batch_tokens, sizeof(int) * b);
  ok = ok && dev_alloc(s, (void**)&s->b_hidden, 4 * b * c.n_embd) && dev_alloc(s, (void**)&s->b_norm, 4 * b * c.n_embd);
  ok = ok && dev_alloc(s, (void**)&s->b_y, 4 * b * c.n_embd);
  ok = ok && dev_alloc(s, (void**)&s->b_q, 4 * b * q_dim) && dev_alloc(s, (void**)&s->b_attn, 4 * b * q_dim);
  ok = ok && dev_alloc(s, (void**)&s->b_k, 4 * b * kv_dim) && dev_alloc(s, (void**)&s->b_v, 4 * b * kv_dim);
  ok = ok && dev_alloc(s, (void**)&s->b_gate, 4 * b * c.n_ff) && dev_alloc(s, (void**)&s->b_up, 4 * b * c.n_ff);
  ok = ok && dev_alloc(s, (void**)&s->b_ffn, 4 * b * c.n_ff);
  ok = ok && dev_alloc(s, (void**)&s->b_partial, sizeof(double) * (size_t)rms_norm_batch_partials(B));
  s->batch_cap = ok ? B : -1;
  return ok;
}

}  // namespace

uint32_t emelb_llama_prefill(emelb_llama* s, const int32_t* tokens, int32_t n, int32_t start_pos) {
  if (!s || !tokens || n <= 0 || !all_bound(s) || start_pos < 0 || start_pos + n > s->cfg.n_ctx) return EMELB_INVALID_REQUEST;
  for (int i = 0; i < n; ++i)
    if (!valid_step(s, tokens[i], start_pos + i)) return EMELB_INVALID_REQUEST;
  emelb_ctx* c = s->c;
  cudaSetDevice(c->device);
  bool ok = true;
  int done = 0;
  const int batch = prefill_batch_size(s, n);
  if (batch > 0 && reserve_batch(s, batch < s->cfg.n_ctx ? batch : s->cfg.n_ctx)) {
    // whole batches, then whatever is left as one shorter batch
    while (ok && n - done >= 2) {
      const int lim = batch < s->batch_cap ? batch : s->batch_cap;
      const int B = n - done < lim ? n - done : lim;
      std::memcpy(s->host_pinned, tokens + done, sizeof(int) * (size_t)B);
      ok = ctx_cuda_ok(c, cudaMemcpyAsync(s->batch_tokens, s->host_pinned, sizeof(int) * (size_t)B, cudaMemcpyHostToDevice, c->stream));
      c->diag.h2d_bytes += sizeof(int) * (uint64_t)B;
      Enqueue e{s, c->stream};
      e.prefill_chunk(B, start_pos + done);
      ok = ok && e.ok && ctx_cuda_ok(c, cudaStreamSynchronize(c->stream));  // host_pinned is reused by the next batch
      c->diag.kernel_launches += e.launches;
      done += B;
    }
    if (!ok) return EMELB_INTERNAL_ERROR;
  }
  if (done < n) {
    if (!step_ready(s, MODE_PREFILL, tokens[done], start_pos + done)) return EMELB_INTERNAL_ERROR;
    for (int i = done; ok && i < n; ++i) {
      ok = ctx_cuda_ok(c, launch_step_begin(s->state, tokens[i], start_pos + i, c->stream));
      ok = ok && step_launch(s, MODE_PREFILL);
    }
    c->diag.kernel_launches += (uint64_t)(n - done);
  }
  ok = ok && ctx_cuda_ok(c, cudaStreamSynchronize(c->stream));
  return ok ? EMELB_OK : EMELB_INTERNAL_ERROR;
}

namespace {

// buffers of the batch step, sized for the session's sequence count
bool free_owned(emelb_llama* s, void* p);

bool reserve_sequences(emelb_llama* s) {
  if (s->seq_cap >= s->n_seq) return true;
  // sized for fewer sequences before: release those buffers first
  for (void* p : {(void*)s->b_qs, (void*)s->b_logits, (void*)s->b_part_acc, (void*)s->b_part_ml, (void*)s->b_out})
    if (p) free_owned(s, p);
  s->b_qs = s->b_logits = s->b_part_acc = s->b_part_ml = nullptr;
  s->b_out = nullptr;
  s->seq_cap = 0;
  const emelb_llama_config& c = s->cfg;
  const size_t b = (size_t)s->n_seq, q_dim = (size_t)c.n_head * c.head_dim;
  bool ok = true;
  if (!s->bstate) {
    ok = dev_alloc(s, (void**)&s->bstate, sizeof(int) * (3 * kMaxSeqs + 4)) && dev_alloc(s, (void**)&s->b_idx, sizeof(int) * kMaxSeqs);
    ok = ok && dev_alloc(s, (void**)&s->b_amax_val, 4 * (size_t)kArgmaxColumnParts * kMaxSeqs) &&
         dev_alloc(s, (void**)&s->b_amax_idx, 4 * (size_t)kArgmaxColumnParts * kMaxSeqs);
  }
  ok = ok && dev_alloc(s, (void**)&s->b_qs, 4 * b * q_dim) && dev_alloc(s, (void**)&s->b_logits, 4 * b * c.n_vocab);
  ok = ok && dev_alloc(s, (void**)&s->b_part_acc, 4 * b * (q_dim / s->G) * s->fa_splits) &&
       dev_alloc(s, (void**)&s->b_part_ml, 4 * b * (c.n_head / s->G) * s->fa_splits * 2);
  ok = ok && dev_alloc(s, (void**)&s->b_out, sizeof(int) * b * (size_t)(c.n_ctx + 8));
  if (ok) s->seq_cap = s->n_seq;
  return ok;
}

// columns of the batch buffers when the batch step is what allocates them: room for the prompt path's batches too
int batch_buffer_columns(const emelb_llama* s) {
  int cols = s->prefill_batch < s->cfg.n_ctx ? s->prefill_batch : s->cfg.n_ctx;
  if (cols < s->n_seq) cols = s->n_seq;
  return cols < 2 ? 2 : cols;
}

void drop_graphs(emelb_llama* s) {
  for (int m = 0; m < MODE_COUNT; ++m) s->graph_attention_mode[m] = -1;
  s->batch_graph_mode = -1;
}

bool free_owned(emelb_llama* s, void* p) {
  for (size_t i = 0; i < s->owned.size(); ++i)
    if (s->owned[i] == p) {
      s->owned.erase(s->owned.begin() + (long)i);
      return cudaFree(p) == cudaSuccess;
    }
  return false;
}

// the batch step needs the batch attention path's preconditions: split-KV attention, room for B columns of the
// widest activation in the context's planes, the communicator in a sharded session
bool batch_step_ok(emelb_llama* s, int B) {
  const emelb_llama_config& c = s->cfg;
  if (s->c->attention_mode != 0 || B < 1 || B > s->n_seq) return false;
  if (s->G > 1 && (!s->c->comm || s->c->comm_world != s->G)) return false;
  int widest = c.n_ff > c.n_embd ? c.n_ff : c.n_embd;
  if (c.n_head * c.head_dim > widest) widest = c.n_head * c.head_dim;
  if ((uint64_t)widest * (uint64_t)B > s->c->act_capacity) return false;
  if (((int64_t)(c.n_head / s->G) * c.head_dim * B) % 256 != 0) return false;   // the merge step works on 256-value groups
  Enqueue probe{s, s->c->stream};
  FlashArgs a = probe.flash_args(0);
  a.heads *= B;
  a.kv_heads *= B;
  return flash_split_supported(a);
}

cudaGraphExec_t batch_step_graph(emelb_llama* s, int B) {
  if (s->batch_graph && s->batch_graph_B == B && s->batch_graph_mode == s->c->attention_mode) return s->batch_graph;
  emelb_ctx* c = s->c;
  if (s->batch_graph) {
    cudaStreamSynchronize(c->stream);
    cudaGraphExecDestroy(s->batch_graph);
    s->batch_graph = nullptr;
  }
  // one eager pass first (sets per-kernel attributes outside the capture); it is a real step for the state the
  // caller has just written, so the KV rows it writes are the rows the replay writes again
  Enqueue warm{s, c->stream};
  warm.batch_step(B);
  if (!warm.ok || !ctx_cuda_ok(c, cudaStreamSynchronize(c->stream))) return nullptr;
  if (!ctx_cuda_ok(c, cudaStreamBeginCapture(c->stream, cudaStreamCaptureModeThreadLocal))) return nullptr;
  Enqueue e{s, c->stream};
  e.batch_step(B);
  cudaGraph_t g = nullptr;
  const bool ended = ctx_cuda_ok(c, cudaStreamEndCapture(c->stream, &g));
  if (!ended || !e.ok || !g) {
    if (g) cudaGraphDestroy(g);
    return nullptr;
  }
  cudaGraphExec_t ex = nullptr;
  const bool inst = ctx_cuda_ok(c, cudaGraphInstantiate(&ex, g, 0));
  cudaGraphDestroy(g);
  if (!inst) return nullptr;
  s->batch_graph = ex;
  s->batch_graph_B = B;
  s->batch_graph_mode = c->attention_mode;
  s->batch_launches = e.launches;
  return ex;
}

bool write_batch_state(emelb_llama* s, const int32_t* tokens, const int32_t* positions, int B) {
  emelb_ctx* c = s->c;
  std::memcpy(s->host_pinned, tokens, sizeof(int) * (size_t)B);
  std::memcpy(s->host_pinned + kMaxSeqs, positions, sizeof(int) * (size_t)B);
  bool ok = ctx_cuda_ok(c, cudaMemcpyAsync(s->bstate, s->host_pinned, sizeof(int) * (size_t)(kMaxSeqs + B), cudaMemcpyHostToDevice, c->stream));
  c->diag.h2d_bytes += sizeof(int) * 2 * (uint64_t)B;
  ok = ok && ctx_cuda_ok(c, launch_batch_begin(s->bstate, kMaxSeqs, B, c->stream));
  c->diag.kernel_launches += 1;
  return ok;
}

bool valid_batch(const emelb_llama* s, const int32_t* tokens, const int32_t* positions, int B, int steps) {
  if (!tokens || !positions || B < 1 || B > s->n_seq || B > kMaxSeqs) return false;
  for (int j = 0; j < B; ++j)
    if (!valid_step(s, tokens[j], positions[j]) || positions[j] + steps > s->cfg.n_ctx) return false;
  return true;
}

// the token-batch buffers were sized by an earlier, smaller batch: release them so that reserve_batch sizes them again
void release_small_batch(emelb_llama* s, int need) {
  if (s->batch_cap <= 0 || s->batch_cap >= need) return;
  cudaStreamSynchronize(s->c->stream);
  for (void* p : {(void*)s->batch_tokens, (void*)s->b_hidden, (void*)s->b_norm, (void*)s->b_y, (void*)s->b_q, (void*)s->b_attn,
                  (void*)s->b_k, (void*)s->b_v, (void*)s->b_gate, (void*)s->b_up, (void*)s->b_ffn, (void*)s->b_partial})
    if (p) free_owned(s, p);
  s->batch_tokens = nullptr;
  s->b_hidden = s->b_norm = s->b_y = s->b_q = s->b_attn = s->b_k = s->b_v = s->b_gate = s->b_up = s->b_ffn = nullptr;
  s->b_partial = nullptr;
  s->batch_cap = 0;
  if (s->batch_graph) {
    cudaGraphExecDestroy(s->batch_graph);
    s->batch_graph = nullptr;
  }
}

}  // namespace

uint32_t emelb_llama_set_sequences(emelb_llama* s, int32_t n_seq) {
  if (!s || n_seq < 1 || n_seq > kMaxSeqs) return EMELB_INVALID_REQUEST;
  emelb_ctx* c = s->c;
  cudaSetDevice(c->device);
  if (!ctx_cuda_ok(c, cudaStreamSynchronize(c->stream))) return EMELB_INTERNAL_ERROR;
  if (n_seq == s->n_seq) return EMELB_OK;
  const emelb_llama_config& g = s->cfg;
  const size_t halves = (size_t)g.n_layer * (size_t)n_seq * (g.n_head_kv / s->G) * s->capacity * g.head_dim;
  __half *k = nullptr, *v = nullptr;
  if (!dev_alloc(s, (void**)&k, 2 * halves)) return EMELB_INTERNAL_ERROR;
  if (!dev_alloc(s, (void**)&v, 2 * halves)) {
    free_owned(s, k);
    return EMELB_INTERNAL_ERROR;
  }
  free_owned(s, s->kcache);
  free_owned(s, s->vcache);
  s->kcache = k;
  s->vcache = v;
  s->n_seq = n_seq;
  s->cur_seq = 0;
  s->token_layers_valid = false;
  drop_graphs(s);
  const bool ok = ctx_cuda_ok(c, cudaMemsetAsync(k, 0, 2 * halves, c->stream)) && ctx_cuda_ok(c, cudaMemsetAsync(v, 0, 2 * halves, c->stream)) &&
                  ctx_cuda_ok(c, cudaStreamSynchronize(c->stream));
  return ok ? EMELB_OK : EMELB_INTERNAL_ERROR;
}

uint32_t emelb_llama_select_sequence(emelb_llama* s, int32_t seq) {
  if (!s || seq < 0 || seq >= s->n_seq) return EMELB_INVALID_REQUEST;
  if (seq != s->cur_seq) {
    s->cur_seq = seq;
    for (int m = 0; m < MODE_COUNT; ++m) s->graph_attention_mode[m] = -1;   // captured steps hold the other sequence's planes
  }
  return EMELB_OK;
}

uint32_t emelb_llama_decode_batch(emelb_llama* s, const int32_t* tokens, const int32_t* positions, int32_t n_seq,
                                  float* logits_out, int32_t* tokens_out) {
  if (!s || !all_bound(s) || !valid_batch(s, tokens, positions, n_seq, 1)) return EMELB_INVALID_REQUEST;
  emelb_ctx* c = s->c;
  cudaSetDevice(c->device);
  if (!batch_step_ok(s, n_seq)) return EMELB_UNSUPPORTED_OP;
  release_small_batch(s, n_seq);
  if (!reserve_sequences(s) || !reserve_batch(s, batch_buffer_columns(s)) || s->batch_cap < n_seq) return EMELB_INTERNAL_ERROR;
  bool ok = write_batch_state(s, tokens, positions, n_seq);
  Enqueue e{s, c->stream};
  if (ok) e.batch_step(n_seq);
  ok = ok && e.ok;
  c->diag.kernel_launches += e.launches;
  const size_t lbytes = sizeof(float) * (size_t)s->cfg.n_vocab * (size_t)n_seq;
  if (ok && logits_out) {
    ok = ctx_cuda_ok(c, cudaMemcpyAsync(logits_out, s->b_logits, lbytes, cudaMemcpyDeviceToHost, c->stream));
    c->diag.d2h_bytes += lbytes;
  }
  if (ok && tokens_out) {
    ok = ctx_cuda_ok(c, cudaMemcpyAsync(s->host_pinned, s->b_idx, sizeof(int) * (size_t)n_seq, cudaMemcpyDeviceToHost, c->stream));
    c->diag.d2h_bytes += sizeof(int) * (uint64_t)n_seq;
  }
  ok = ok && ctx_cuda_ok(c, cudaStreamSynchronize(c->stream));
  if (ok && tokens_out) std::memcpy(tokens_out, s->host_pinned, sizeof(int) * (size_t)n_seq);
  return ok ? EMELB_OK : EMELB_INTERNAL_ERROR;
}

uint32_t emelb_llama_generate_batch(emelb_llama* s, const int32_t* first_tokens, const int32_t* start_positions, int32_t n_seq,
                                    int32_t n_steps, int32_t* tokens_out) {
  if (!s || !tokens_out || n_steps <= 0 || !all_bound(s) || !valid_batch(s, first_tokens, start_positions, n_seq, n_steps))
    return EMELB_INVALID_REQUEST;
  emelb_ctx* c = s->c;
  cudaSetDevice(c->device);
  if (!batch_step_ok(s, n_seq)) return EMELB_UNSUPPORTED_OP;
  release_small_batch(s, n_seq);
  if (!reserve_sequences(s) || !reserve_batch(s, batch_buffer_columns(s)) || s->batch_cap < n_seq) return EMELB_INTERNAL_ERROR;
  bool ok = write_batch_state(s, first_tokens, start_positions, n_seq);
  cudaGraphExec_t g = ok && !s->streamed ? batch_step_graph(s, n_seq) : nullptr;
  if (!g && !(ok && s->streamed)) return EMELB_INTERNAL_ERROR;
  for (int i = 0; ok && i < n_steps; ++i) {
    if (g) {
      ok = ctx_cuda_ok(c, cudaGraphLaunch(g, c->stream));
    } else {
      // streamed layers: plain launches, the window's events order the slot copies
      Enqueue e{s, c->stream};
      e.batch_step(n_seq);
      ok = e.ok;
      s->batch_launches = e.launches;
    }
    ok = ok && ctx_cuda_ok(c, launch_batch_advance(s->bstate, kMaxSeqs, n_seq, s->b_idx, s->b_out, c->stream));
  }
  c->diag.kernel_launches += (uint64_t)n_steps * (uint64_t)(s->batch_launches + 1);
  const size_t bytes = sizeof(int) * (size_t)n_steps * (size_t)n_seq;
  ok = ok && ctx_cuda_ok(c, cudaMemcpyAsync(tokens_out, s->b_out, bytes, cudaMemcpyDeviceToHost, c->stream));
  ok = ok && ctx_cuda_ok(c, cudaStreamSynchronize(c->stream));
  c->diag.d2h_bytes += bytes;
  return ok ? EMELB_OK : EMELB_INTERNAL_ERROR;
}

uint32_t emelb_llama_batch_launches_per_step(const emelb_llama* s, int32_t* out) {
  if (!s || !out) return EMELB_INVALID_REQUEST;
  *out = s->batch_launches + 1;
  return EMELB_OK;
}

uint32_t emelb_llama_generate(emelb_llama* s, int32_t first_token, int32_t start_pos, int32_t n, int32_t* tokens_out) {
  if (!s || !tokens_out || n <= 0 || !all_bound(s) || !valid_step(s, first_token, start_pos) || start_pos + n > s->cfg.n_ctx)
    return EMELB_INVALID_REQUEST;
  emelb_ctx* c = s->c;
  cudaSetDevice(c->device);
  if (!step_ready(s, MODE_ARGMAX, first_token, start_pos)) return EMELB_INTERNAL_ERROR;
  bool ok = ctx_cuda_ok(c, launch_step_begin(s->state, first_token, start_pos, c->stream));
  for (int i = 0; ok && i < n; ++i) ok = step_launch(s, MODE_ARGMAX);
  c->diag.kernel_launches += 1;
  ok = ok && ctx_cuda_ok(c, cudaMemcpyAsync(s->host_pinned, s->tokens_dev, sizeof(int) * (size_t)n, cudaMemcpyDeviceToHost, c->stream));
  ok = ok && ctx_cuda_ok(c, cudaStreamSynchronize(c->stream));
  if (!ok) return EMELB_INTERNAL_ERROR;
  c->diag.d2h_bytes += sizeof(int) * (uint64_t)n;
  std::memcpy(tokens_out, s->host_pinned, sizeof(int) * (size_t)n);
  return EMELB_OK;
}

uint32_t emelb_llama_exchange_export(emelb_llama* s, uint8_t* handle_out, uint64_t handle_bytes) {
  if (!s || !handle_out || handle_bytes < EMELB_EXCHANGE_HANDLE_BYTES || s->G <= 1 || !s->arena) return EMELB_INVALID_REQUEST;
  static_assert(sizeof(cudaIpcMemHandle_t) <= EMELB_EXCHANGE_HANDLE_BYTES, "handle buffer too small");
  cudaSetDevice(s->c->device);
  // the arena must be zero before any peer can see it
  if (!ctx_cuda_ok(s->c, cudaStreamSynchronize(s->c->stream))) return EMELB_INTERNAL_ERROR;
  cudaIpcMemHandle_t h;
  if (!ctx_cuda_ok(s->c, cudaIpcGetMemHandle(&h, s->arena))) return EMELB_INTERNAL_ERROR;
  std::memset(handle_out, 0, EMELB_EXCHANGE_HANDLE_BYTES);
  std::memcpy(handle_out, &h, sizeof h);
  return EMELB_OK;
}

uint32_t emelb_llama_exchange_attach(emelb_llama* s, const uint8_t* handles, uint64_t handles_bytes) {
  if (!s || !handles || s->G <= 1 || s->G > kMaxPeers || handles_bytes < (uint64_t)s->G * EMELB_EXCHANGE_HANDLE_BYTES || s->peers_attached)
    return EMELB_INVALID_REQUEST;
  cudaSetDevice(s->c->device);
  for (int g = 0; g < s->G; ++g) {
    if (g == s->rank) continue;
    cudaIpcMemHandle_t h;
    std::memcpy(&h, handles + (size_t)g * EMELB_EXCHANGE_HANDLE_BYTES, sizeof h);
    void* p = nullptr;
    if (!ctx_cuda_ok(s->c, cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess))) return EMELB_INTERNAL_ERROR;
    s->peer_base[g] = static_cast<char*>(p);
  }
  // descriptors of the joins that run inside kernels: one flag row, sequence counter and block counter per join of
  // a layer (row 0 belongs to the stand-alone join kernel)
  {
    const emelb_llama_config& c = s->cfg;
    const size_t q_l = (size_t)(c.n_head / s->G) * c.head_dim, embd_l = (size_t)c.n_embd / s->G, ff_l = (size_t)c.n_ff / s->G;
    JoinOut jo[5] = {};
    JoinIn ji[5] = {};
    for (int id = 1; id <= 4; ++id) {
      for (int g = 0; g < s->G; ++g) jo[id].base[g] = s->peer_base[g];
      jo[id].flag_offset = (unsigned)(s->flags_off + 32 * (size_t)id);
      jo[id].seq = reinterpret_cast<unsigned*>(s->arena + s->seq_off) + id;
      jo[id].done = reinterpret_cast<int*>(s->arena + s->seq_off + 64) + id;
      jo[id].world = s->G;
      jo[id].rank = s->rank;
      ji[id].flags = reinterpret_cast<const unsigned*>(s->arena + s->flags_off + 32 * (size_t)id);
      ji[id].seq = jo[id].seq;
      ji[id].world = s->G;
      ji[id].rank = s->rank;
      ji[id].wait_ns = s->c->peer_wait_ns;
    }
    auto planes_of = [&](JoinOut& j, const ActPlanesMut& pl, size_t per_rank) {
      j.qs_offset = reinterpret_cast<const char*>(pl.qs) - s->arena;
      j.bsums_offset = reinterpret_cast<const char*>(pl.bsums) - s->arena;
      j.d_offset = reinterpret_cast<const char*>(pl.d) - s->arena;
      j.first_block = (int)((size_t)s->rank * per_rank / QK_K);
    };
    planes_of(jo[1], s->attn_planes, q_l);                                        // J_ATTN
    planes_of(jo[3], s->ffn_planes, ff_l);                                        // J_FFN
    jo[2].out_offset = jo[4].out_offset = (int64_t)(reinterpret_cast<char*>(s->hidden + s->rank * embd_l) - s->arena);   // J_HIDDEN_A / _B
    bool ok = s->join_out_dev || (dev_alloc(s, (void**)&s->join_out_dev, sizeof jo) && dev_alloc(s, (void**)&s->join_in_dev, sizeof ji));
    ok = ok && ctx_cuda_ok(s->c, cudaMemcpy(s->join_out_dev, jo, sizeof jo, cudaMemcpyHostToDevice)) &&
         ctx_cuda_ok(s->c, cudaMemcpy(s->join_in_dev, ji, sizeof ji, cudaMemcpyHostToDevice));
    if (!ok) return EMELB_INTERNAL_ERROR;
  }
  s->peers_attached = true;
  for (int m = 0; m < MODE_COUNT; ++m) s->graph_attention_mode[m] = -1;   // captured steps hold the NCCL joins
  return EMELB_OK;
}

uint32_t emelb_llama_exchange_detach(emelb_llama* s) {
  if (!s) return EMELB_INVALID_REQUEST;
  cudaSetDevice(s->c->device);
  if (!ctx_cuda_ok(s->c, cudaStreamSynchronize(s->c->stream))) return EMELB_INTERNAL_ERROR;
  for (int g = 0; g < kMaxPeers; ++g)
    if (s->peer_base[g] && g != s->rank) {
      cudaIpcCloseMemHandle(s->peer_base[g]);
      s->peer_base[g] = nullptr;
    }
  if (s->peers_attached)
    for (int m = 0; m < MODE_COUNT; ++m) s->graph_attention_mode[m] = -1;   // captured steps hold the peer pointers
  s->peers_attached = false;
  cudaGetLastError();
  return EMELB_OK;
}

uint32_t emelb_llama_decode_profile(emelb_llama* s, int32_t token, int32_t position, uint64_t* stamps_ns, uint64_t stamps_count) {
  if (!s || !stamps_ns || !valid_step(s, token, position) || !all_bound(s)) return EMELB_INVALID_REQUEST;
  const uint64_t need = (uint64_t)s->cfg.n_layer * kTokenTracePoints;
  if (stamps_count < need) return EMELB_INVALID_REQUEST;
  emelb_ctx* c = s->c;
  cudaSetDevice(c->device);
  prepare_token_kernel(s);
  if (!s->token_usable || c->attention_mode != 0) return EMELB_UNSUPPORTED_OP;
  if (!s->token_trace && !dev_alloc(s, (void**)&s->token_trace, need * sizeof(unsigned long long))) return EMELB_INTERNAL_ERROR;
  bool ok = ctx_cuda_ok(c, cudaMemsetAsync(s->token_trace, 0, need * sizeof(unsigned long long), c->stream));
  ok = ok && ctx_cuda_ok(c, launch_step_begin(s->state, token, position, c->stream));
  ok = ok && ctx_cuda_ok(c, launch_embed_row(s->tok_embd.type, s->tok_embd.dev, s->tok_embd.row_bytes, s->state, s->hidden, s->cfg.n_embd, c->stream));
  TokenArgs a = token_args(s);
  a.trace = s->token_trace;
  ok = ok && ctx_cuda_ok(c, launch_llama_token(a, c->sm_count, &s->token_launch, c->stream));
  ok = ok && ctx_cuda_ok(c, cudaMemcpyAsync(stamps_ns, s->token_trace, need * sizeof(unsigned long long), cudaMemcpyDeviceToHost, c->stream));
  ok = ok && ctx_cuda_ok(c, cudaStreamSynchronize(c->stream));
  c->diag.kernel_launches += 3;
  return ok ? EMELB_OK : EMELB_INTERNAL_ERROR;
}

uint32_t emelb_llama_set_prefill_batch(emelb_llama* s, int32_t max_tokens) {
  if (!s || max_tokens < 0) return EMELB_INVALID_REQUEST;
  s->prefill_batch = max_tokens == 1 ? 0 : max_tokens;   // a batch of one is the token-by-token walk
  return EMELB_OK;
}

uint32_t emelb_llama_set_join_fusion(emelb_llama* s, int32_t on) {
  if (!s || (on != 0 && on != 1)) return EMELB_INVALID_REQUEST;
  if (s->fused_joins != (on == 1)) {
    s->fused_joins = on == 1;
    for (int m = 0; m < MODE_COUNT; ++m) s->graph_attention_mode[m] = -1;   // captured steps hold the other joins
  }
  return EMELB_OK;
}

uint32_t emelb_llama_set_step_mode(emelb_llama* s, int32_t mode) {
  if (!s || mode < 0 || mode > 1) return EMELB_INVALID_REQUEST;
  if (s->step_mode != mode)
    for (int m = 0; m < MODE_COUNT; ++m) s->graph_attention_mode[m] = -1;   // captured steps hold the other route
  s->step_mode = mode;
  return EMELB_OK;
}

uint32_t emelb_llama_launches_per_token(const emelb_llama* s, int32_t* out) {
  if (!s || !out) return EMELB_INVALID_REQUEST;
  *out = s->launches_per_token;
  return EMELB_OK;
}

}  // extern "C"
