// Host-side launch interface of the sm_100a kernels (internal to the library;
// the public surface is include/emelb.h).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "common.cuh"

namespace emelb {

// kernel launch, optionally with the programmatic-stream-serialization attribute
template <class... KArgs, class... Args>
inline cudaError_t launch_kernel(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, bool pdl,
                                 Args... args) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

// set by the decoder while it enqueues a token step: launches made through EMELB_LAUNCH then carry the
// programmatic-stream-serialization attribute (every such kernel begins with pdl_trigger(); pdl_wait();)
extern thread_local bool g_pdl_launch;
#define EMELB_LAUNCH(kern, grid, block, smem, st, ...) \
  ::emelb::launch_kernel(kern, dim3(grid), dim3(block), smem, st, ::emelb::g_pdl_launch, __VA_ARGS__)

constexpr int kMaxArgmaxParts = 2048;

constexpr int kSchedSlots = 64;   // task-counter slots rotated over consecutive mat-vec launches

// ---- joins of row intervals by peer stores, fused into the kernels either side of the join (same node, one
// rank per GPU).  The producing kernel writes its output rows into every rank's copy of the vector (the
// exchange arenas hold it at the same offset) and its last block raises this rank's flag on every peer with the
// join's new sequence number; the consuming kernel waits, bounded, until every peer's flag has reached this
// rank's own sequence number before it reads the vector.  Plain peer stores and loads only.  The descriptors live
// in device memory (a session writes them once when its peers are attached); kernels take pointers to them.
constexpr int kMaxPeers = 8;
struct JoinOut {
  char* base[kMaxPeers];   // every rank's exchange arena as mapped here (base[rank] is this rank's own)
  int64_t out_offset;      // f32 output: byte offset inside the arena of the first element this rank produces
  // Q8_K output (the producer quantizes its interval once, every rank's next product reads the planes): byte
  // offsets inside the arena of the full vector's planes, and the first 256-block this rank produces
  int64_t qs_offset, bsums_offset, d_offset;
  int first_block;
  unsigned flag_offset;    // byte offset inside the arena of the join's flag row (one u32 per sender)
  unsigned* seq;           // this rank's sequence counter of the join
  int* done;               // finished-block counter, zero between launches (kernels without one of their own)
  int world, rank;         // world <= 1: no join, a plain local store
};
struct JoinIn {
  const unsigned* flags;   // this rank's copy of the join's flag row; null: nothing to wait for
  const unsigned* seq;     // this rank's sequence counter of the join: the value every peer's flag must reach
  int world, rank;
  unsigned long long wait_ns;
};

struct GemvArgs {
  const uint8_t* W;      // {K, M} native block rows
  int64_t row_bytes;
  int M;
  int K;
  ActPlanes act;         // quantized activations, column planes
  int col0;              // first activation column this launch covers
  float* y;              // y[row*ldy + col]
  int64_t ldy;
  const float* residual; // optional: y = residual + W x  (same indexing as y)
  // up to two more matrices of the same type and K multiplied by the same activations in the same
  // launch (Q/K/V, gate/up): rows of segment s go to ys[s]; M2 = M3 = 0 when unused
  const uint8_t* W2;
  const uint8_t* W3;
  int M2, M3;
  float* y2;
  float* y3;
  // optional fused epilogue of the one-column streaming kernel for a grouped Q/K/V launch (segments 0/1/2):
  // rotate q and k at the device-resident position (adjacent pairs only) and store k, v as f16 KV-cache rows —
  // the RoPE / KV-store step of the layer without its own launch
  const float* rope_cos;   // null: plain f32 outputs
  const float* rope_sin;
  const int* rope_pos;
  int rope_head_dim, rope_rot_dim;
  int rope_seg0;           // which of Q / K / V the launch's first matrix is (a group split by weight type)
  __half* rope_kcache;     // this layer's cache planes, [kv head][capacity][head_dim]
  __half* rope_vcache;
  int64_t rope_cache_head_stride;
  // optional fused prologue of the one-column streaming kernel (K-quant weights only): instead of reading
  // `act`, every CTA normalises pro_x itself, out = (x * 1/sqrt(mean(x^2) + eps)) * pro_w, and quantizes it to
  // Q8_K in shared memory — the rms_norm step of the layer without its own launch
  // pro_w == null: no normalisation, the f32 vector is quantized as it is
  const float* pro_x;
  const float* pro_w;
  float pro_eps;
  // one-column plain products of a row-sharded session: wait for join_in before reading pro_x or the planes,
  // and / or write the f32 rows (ldy == 1, first matrix only) to every rank and raise join_out
  const JoinIn* join_in;     // device memory; null: none
  const JoinOut* join_out;   // device memory; null: none
  uint8_t* tc_ws;        // workspace of the many-column tensor-core kernel (null: that kernel is not used)
  size_t tc_ws_bytes;
  int tc_ws_reuse;       // the previous many-column Q4_K product of this stream used the same planes, K, columns and col0
  int* sched;            // {next task, finished blocks}: zero between launches (self-rearming)
  int* status;           // optional: set to 1 by a kernel whose bounded wait ran out
  int pdl;               // launch with programmatic stream serialization (kernels wait before dependent reads)
  float* part_val;       // argmax: per-block candidates (kMaxArgmaxParts)
  int* part_idx;
  float* best_val;       // argmax result
  int* best_idx;
};

// gemv.cu
bool gemv_fast_path_ok(int type, const void* w, int64_t row_bytes, int K);
cudaError_t launch_gemv(int type, const GemvArgs& a, int ncols, bool argmax, int sm_count, cudaStream_t st,
                        int* launches);
// whether launch_gemv (without argmax) hands this product to the tcgen05 kernel
bool gemv_takes_tensor_core(int type, const GemvArgs& a, int ncols);

// gemm_q8_mma.cu: 32 and more columns of Q8_0 / Q4_0 weights (mma.sync int8, one block per instruction)
bool gemm_q8_mma_supported(int type, const GemvArgs& a, int ncols);
cudaError_t launch_gemm_q8_mma(int type, const GemvArgs& a, int ncols, int sm_count, cudaStream_t st);

// gemm_q4k_mma.cu: 5 to 31 columns of Q4_K weights (mma.sync int8, one sub-block per instruction)
bool gemm_q6k_mma_supported(int type, const GemvArgs& a, int ncols);
cudaError_t launch_gemm_q6k_mma(const GemvArgs& a, int ncols, int sm_count, cudaStream_t st);
bool gemm_q4k_mma_supported(int type, const GemvArgs& a, int ncols);
cudaError_t launch_gemm_q4k_mma(const GemvArgs& a, int ncols, int sm_count, cudaStream_t st);

// gemv2.cu
cudaError_t launch_gemv_stream2(int type, const GemvArgs& a, int ncols, bool argmax, int sm_count, cudaStream_t st,
                                int* launches, int* grid_out);

cudaError_t launch_argmax_f32(const float* x, int n, float* out_val, int* out_idx, cudaStream_t st);

// quantize.cu — built with -fmad=false: every float op rounds as written
struct ActPlanesMut {
  int8_t* qs;
  float* d;
  int16_t* bsums;
};
// x: f32 {n, K} token-fastest (x[p*n + j]); quantizes columns [0, ncols) into planes 0..ncols-1
cudaError_t launch_quantize_q8_k_planes(const float* x, int n, int ncols, int K, ActPlanesMut out, cudaStream_t st);
cudaError_t launch_quantize_q8_0_planes(const float* x, int n, int ncols, int K, ActPlanesMut out, cudaStream_t st);
// reference array-of-blocks output: row j of `out` (row_bytes apart) = column j
cudaError_t launch_quantize_q8_k_blocks(const float* x, int n, int K, uint8_t* out, int64_t row_bytes, cudaStream_t st);
cudaError_t launch_quantize_q8_0_blocks(const float* x, int n, int K, uint8_t* out, int64_t row_bytes, cudaStream_t st);
// reference blocks (one vector of K) -> planes
cudaError_t launch_blocks_to_planes(int type, const uint8_t* blocks, int K, ActPlanesMut out, cudaStream_t st);
// src rows of native blocks -> f32 rows
cudaError_t launch_dequantize(int type, const uint8_t* src, int64_t src_row_bytes, float* dst, int64_t dst_row_elems,
                              int K, int M, cudaStream_t st);

// elementwise.cu — the steps between the matrix products of a decoder layer
// family: 0 = f32 output only, 1 = also Q8_K planes, 2 = also Q8_0 planes
cudaError_t launch_rms_norm(const float* x, const float* w, float eps, int n, float* out, int family, ActPlanesMut planes,
                            cudaStream_t st);
cudaError_t launch_rope_store(float* q, const float* k, const float* v, const float* cos_t, const float* sin_t,
                              const int* pos_dev, int n_head, int n_head_kv, int head_dim, int rot_dim, int neox,
                              __half* kcache, __half* vcache, int64_t cache_head_stride, cudaStream_t st);
// join: the product of this rank's n elements (a multiple of 256) goes, quantized to Q8_K, into every rank's planes
cudaError_t launch_swiglu_join(const float* gate, const float* up, int n, const JoinOut* join_dev, cudaStream_t st);
cudaError_t launch_swiglu(const float* gate, const float* up, int n, float* out, int family, ActPlanesMut planes,
                          cudaStream_t st);
cudaError_t launch_embed_row(int type, const uint8_t* table, int64_t row_bytes, const int* token_dev, float* dst, int K,
                             cudaStream_t st);
// token batches (prompt processing): activations feature-major, element e of token j at x[e * B + j]
cudaError_t launch_embed_rows(int type, const uint8_t* table, int64_t row_bytes, const int* tokens_dev, int B, float* dst,
                              int K, cudaStream_t st);
// partial: scratch of rms_norm_batch_partials(B) doubles
cudaError_t launch_rms_norm_batch(const float* x, const float* w, float eps, int K, int B, float* out, double* partial,
                                  cudaStream_t st);
int rms_norm_batch_partials(int B);
cudaError_t launch_rope_store_batch(float* q, const float* k, const float* v, const float* cos_t, const float* sin_t, int pos0,
                                    int B, int n_head, int n_head_kv, int head_dim, int rot_dim, int neox, __half* kcache,
                                    __half* vcache, int64_t cache_head_stride, cudaStream_t st);
cudaError_t launch_add_inplace(float* acc, const float* y, int64_t n, cudaStream_t st);
// ---- one decode step of B sequences together (activations {features, B}, sequence index fastest)
// state: three rows of `stride` ints {token, position, kv token count} per sequence, then {step}
cudaError_t launch_batch_begin(int* state, int stride, int B, cudaStream_t st);
// rotates q column j at positions[j] into q_out [B][n_head * head_dim] and writes k, v column j as f16 rows of
// sequence j's cache (cache planes of consecutive sequences lie seq_stride halves apart)
cudaError_t launch_rope_store_seqs(const float* q, const float* k, const float* v, const float* cos_t, const float* sin_t,
                                   const int* positions, int B, int n_head, int n_head_kv, int head_dim, int rot_dim, int neox,
                                   float* q_out, __half* kcache, __half* vcache, int64_t seq_stride, int64_t cache_head_stride,
                                   cudaStream_t st);
// rms_norm of every column of x {K, B} and its Q8_K planes in one launch (a few columns: one CTA each)
cudaError_t launch_rms_norm_quant_cols(const float* x, const float* w, float eps, int K, int B, ActPlanesMut planes, cudaStream_t st);
// SwiGLU of gate, up {K, B} quantized to Q8_K planes in one launch (a few columns)
cudaError_t launch_swiglu_quant_cols(const float* gate, const float* up, int K, int B, ActPlanesMut planes, cudaStream_t st);
// per column of x {rows, B}: the highest value and, on ties, the lowest row (src/emel/kernel/detail.hpp:3720-3723)
constexpr int kArgmaxColumnParts = 256;
cudaError_t launch_argmax_columns(const float* x, int rows, int B, float* part_val, int* part_idx, int* out_idx, cudaStream_t st);
// token <- idx, position and token count + 1, idx appended to out[step * B + j]
cudaError_t launch_batch_advance(int* state, int stride, int B, const int* idx, int* out, cudaStream_t st);
// causal attention of a batch of B query tokens at positions pos0 .. pos0 + B - 1 over the f16 KV cache
// (q, dst feature-major {heads * head_dim, B}; f32 online softmax); false from the predicate: not taken
struct PrefillAttnArgs {
  const float* q;
  float* dst;
  const __half* k;   // one layer's cache: [kv_head][position][head_dim]
  const __half* v;
  int64_t cache_head_stride;  // halves
  int head_dim, heads, kv_heads, B, pos0;
  float scale;
};
bool prefill_attention_supported(const PrefillAttnArgs& a);
cudaError_t launch_prefill_attention(const PrefillAttnArgs& a, cudaStream_t st);
// op_rms_norm / op_rope as stand-alone ops over strided f32 tensors (byte strides, up to 4 dims)
struct StridedF32 {
  char* base;
  int64_t ne[4];
  int64_t nb[4];
};
cudaError_t launch_rms_norm_rows(const StridedF32& src, const StridedF32& dst, float eps, cudaStream_t st);
// positions: i32, element i2 at pos_base + i2 * pos_stride; theta_scale = powf(freq_base, -2 / n_dims) from the host libm
cudaError_t launch_rope_rows(const StridedF32& src, const StridedF32& dst, const char* pos_base, int64_t pos_stride, int n_dims,
                             int neox, float theta_scale, float freq_scale, float attn_factor, cudaStream_t st);
// state = {token, position, kv_tokens, step}
cudaError_t launch_step_begin(int* state, int token, int position, cudaStream_t st);
cudaError_t launch_step_advance(int* state, const int* best_idx, int* tokens_out, cudaStream_t st);

// gemm_tc.cu — Q4_K x Q8_K for many columns on the tensor cores (tcgen05, TMEM accumulators);
// same numbers as the mat-vec kernels.  a.col0/a.y/a.ldy address the output as for launch_gemv.
constexpr int kGemmTcMinCols = 32;
constexpr int kGemmMmaMinCols = 9;   // Q6_K: fewer columns run the CUDA-core mat-vec kernels
constexpr int kGemmQ4kMmaMinCols = 5; // Q4_K: 8 columns take 39 / 63 us through the mat-vec kernel, 23-28 / 35 us through the mma.sync one (4096x14336 / 14336x4096)
constexpr int kGemmQ8MmaMinCols = 3; // Q8_0 / Q4_0: from three columns on the mma.sync kernel (21-24 us for up to 8 columns of 14336x4096) beats the mat-vec kernels (29 us at 4 columns)
bool gemm_tc_supported(int type, int K, int ncols, const void* W, int64_t row_bytes, const ActPlanes& act);
// true when launch_gemv would run the kernel that honours GemvArgs::pro_x for this matrix
bool gemv_prologue_supported(int type, const void* w, int64_t row_bytes, int K);
size_t gemm_tc_workspace_bytes(int K, int ncols);
cudaError_t launch_gemm_q4k_tc(const GemvArgs& a, int ncols, int sm_count, uint8_t* workspace, cudaStream_t st);

cudaError_t launch_argmax_pair_store(const float* best_val, const int* best_idx, int row_offset, int* pair, cudaStream_t st);
cudaError_t launch_argmax_pair_finish(const int* pairs, int n, float* out_val, int* out_idx, cudaStream_t st);

// comm.cu — join of row intervals by peer stores (one rank per GPU, same node)
struct PeerGatherArgs {
  char* local_base;            // this rank's arena
  char* peer_base[kMaxPeers];  // every rank's arena as mapped here (own entry = local_base)
  size_t offset_bytes;         // of this rank's interval inside the arena (vector offset + rank * bytes_per_rank)
  size_t bytes_per_rank;
  size_t flags_offset;         // kMaxPeers u32 sequence flags inside the arena, indexed by sender
  unsigned int* seq;           // this rank's join counter
  int rank, world;
  int* status;
  unsigned long long wait_ns;  // how long the kernel waits for the peers' flags before it gives up
};
constexpr unsigned long long kPeerWaitNsDefault = 10000000000ull;  // 10 s: covers host-side skew between the ranks' launches
cudaError_t launch_peer_gather(const PeerGatherArgs& a, cudaStream_t st);

// token_kernel.cu — one decode token (all layers) as one persistent kernel
struct TokenLayerW {       // one layer's weights (device pointers; Q4_K matrices, f32 norm vectors)
  const uint8_t *wq, *wk, *wv, *wo, *gate, *up, *down;
  const float *attn_norm, *ffn_norm;
};
struct TokenArgs {
  const TokenLayerW* layers;   // device array, n_layer entries
  int n_layer, n_embd, n_ff, heads, kv_heads, head_dim;
  float eps;
  const int* state;            // {token, position, kv_tokens, step}
  float *hidden, *q, *ffn;     // f32 vectors: residual stream, rotated queries, SwiGLU product
  ActPlanesMut attn_planes;    // attention context quantized for the output projection
  float* attn_f32;             // optional f32 copy of the attention context
  __half *kcache, *vcache;     // [layer][kv_head][capacity][head_dim]
  int64_t capacity;
  const float *rope_cos, *rope_sin;
  int rope_rot_dim;
  float attn_scale;
  int fa_splits;               // KV ranges per KV head (the stand-alone split kernel's choice)
  float *part_acc, *part_ml;   // split partials (FlashArgs layout)
  int* kv_cnt;                 // one arrival counter per (KV head, query-head quad): zero between launches
  float* bv_table;             // block-value table and row-group counters of the products
  int* grp_cnt;
  unsigned* bar;               // grid barrier {arrivals, generation, abort}: arrivals and abort zero between launches
  int* status;
  unsigned long long* trace;   // optional: CTA 0 stamps %globaltimer at 16 points per layer (phase profile)
};
constexpr int kTokenTracePoints = 16;
struct TokenLaunchState {      // per session, host side
  size_t smem = 0;
};
size_t llama_token_smem_bytes(int n_embd, int n_ff);
bool llama_token_supported(const TokenArgs& a, int attention_splits, int n_ctx);
cudaError_t launch_llama_token(const TokenArgs& a, int sm_count, TokenLaunchState* state, cudaStream_t st);

// synth.cu — synthetic N(0, sigma) data generated and block-encoded on the device
cudaError_t launch_fill_normal(float* out, uint64_t n, uint64_t seed, float sigma, uint64_t offset, cudaStream_t st);
cudaError_t launch_encode_normal(int type, uint8_t* out, uint64_t elems, uint64_t seed, float sigma, uint64_t offset,
                                 cudaStream_t st);

// attention.cu
struct FlashArgs {
  const float* q;        // {d, 1, H} dense
  const __half* k;       // {d, T, Hkv}, byte strides nb1 / nb2
  const __half* v;
  float* dst;            // {d, 1, H} dense
  int64_t k_nb1, k_nb2, v_nb1, v_nb2;
  int head_dim, heads, kv_heads;
  int tokens;            // used when tokens_dev == nullptr
  const int* tokens_dev; // optional: token count read on the device (graph replay)
  float scale;
  int splits;            // KV splits per kv head
  float* part_acc;       // [H][splits][d]
  float* part_ml;        // [H][splits][2]  (running max, running sum)
  // several sequences at once (one query token each): sequence i owns kv heads [i * kv_heads_per_seq, ...) of the
  // cache planes and the matching query heads, and tokens_dev[i] is its token count; 0: one sequence
  int kv_heads_per_seq;
  int dst_seqs;          // > 1: dst is {heads_per_seq * d, dst_seqs} with the sequence index fastest (a product's activation layout)
  const JoinOut* join_out;   // device memory or null; split-KV merge step: this rank's heads, quantized to Q8_K, go into every rank's planes
};
// out_family 1 / 2: the merge step also writes the result quantized (Q8_K / Q8_0 planes, one column) for the
// matrix product that consumes it; only when flash_merge_can_quantize(a)
cudaError_t launch_flash_decode(const FlashArgs& a, int sm_count, cudaStream_t st, int* launches, int out_family,
                                ActPlanesMut out_planes);
bool flash_merge_can_quantize(const FlashArgs& a);
// attention_bf16.cu: kernel::attention's head-range event (bf16 KV ring buffer, reference scalar arithmetic)
struct HeadRangeArgs {
  const float* query;
  const uint16_t* key;
  const uint16_t* value;
  float* output;
  size_t layer_offset;
  int hidden_dim, head_dim, head_begin, head_end, capacity, physical_begin, valid;
  float scale;   // 1 / sqrt(head_dim), computed on the host as the reference does
};
cudaError_t launch_head_range_attention(const HeadRangeArgs& a, cudaStream_t st);
// score_ws: [heads][t_stride] f32 scratch; order 1 = scalar route, 2 = x86 AVX2 route
cudaError_t launch_flash_reference_order(const FlashArgs& a, float* score_ws, int t_stride, int order, cudaStream_t st,
                                         int* launches);
// true when the split-KV kernel takes this request (head_dim 64/128, 16-byte aligned rows)
bool flash_split_supported(const FlashArgs& a);
int flash_pick_splits(int tokens, int kv_heads, int sm_count, int max_splits);

}  // namespace emelb
