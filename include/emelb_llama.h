/*
 * emelb_llama.h — device-resident Llama-architecture decode loop over the
 * kernels of emelb.h.
 *
 * Restates the caller side of the hot path: the reference's generator issues,
 * per token, the embedding row copy, per layer rms_norm -> Q/K/V mat-vecs ->
 * RoPE -> f16 KV store -> flash attention -> output projection + residual ->
 * rms_norm -> gate/up mat-vecs -> SwiGLU -> down projection + residual, then
 * the output norm and the logits mat-vec
 * (src/emel/text/generator/detail.hpp:3746-3840 compute_layer_attention_residual,
 *  :3852-3926 compute_layer_feed_forward, :3997-4033 compute_logits,
 *  :4860-4914 run_decode).  Here the whole token step is enqueued on the
 * context's stream (captured once as a CUDA graph) with every intermediate
 * kept in HBM; only the token id goes in and the next token id (or the logits)
 * comes out.
 */
#ifndef EMELB_LLAMA_H
#define EMELB_LLAMA_H

#include "emelb.h"
#include "emelb_window.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct emelb_llama_config {
  int32_t n_layer;
  int32_t n_embd;
  int32_t n_head;
  int32_t n_head_kv;
  int32_t head_dim;
  int32_t n_ff;
  int32_t n_vocab;
  int32_t n_ctx;
  int32_t rope_dim;        /* rotated dims per head (n_rot) */
  int32_t rope_neox;       /* 0: adjacent pairs (Llama), 1: half-split pairs
                              (src/emel/text/generator/detail.hpp:38-50) */
  float rope_freq_base;
  float rms_eps;
  int32_t kv_block;        /* KV capacity is n_ctx rounded up to this (16 in the
                              reference, src/emel/memory/view.hpp:18,47-56) */
  int32_t shard_rank;      /* row sharding across GPUs: this rank ... */
  int32_t shard_count;     /* ... of this many (1 = unsharded).  With G > 1 the
                              context must have joined a G-rank exchange group
                              (emelb_comm_init) as this rank; n_head_kv, n_embd,
                              n_ff and n_vocab must be multiples of G; each
                              matrix is bound as this rank's contiguous row
                              interval (M/G rows: whole query/KV heads for
                              Q/K/V), the embedding table and norms whole.
                              Every rank calls decode/prefill/generate with
                              the same arguments; results are identical on
                              all ranks and equal to the unsharded session's
                              (src/emel/kernel/matmul/detail.hpp:36-57). */
} emelb_llama_config;

/* tensor roles for emelb_llama_bind; layer = -1 for the three model-level ones */
enum {
  EMELB_T_TOKEN_EMBD = 0,
  EMELB_T_OUTPUT_NORM = 1,
  EMELB_T_OUTPUT = 2,
  EMELB_T_ATTN_NORM = 3,
  EMELB_T_ATTN_Q = 4,
  EMELB_T_ATTN_K = 5,
  EMELB_T_ATTN_V = 6,
  EMELB_T_ATTN_OUT = 7,
  EMELB_T_FFN_NORM = 8,
  EMELB_T_FFN_GATE = 9,
  EMELB_T_FFN_UP = 10,
  EMELB_T_FFN_DOWN = 11
};

typedef struct emelb_llama emelb_llama;

/* pure check of a configuration (no device needed): EMELB_OK or
 * EMELB_INVALID_REQUEST.  Beyond the plain range checks, a sharded layout
 * (shard_count G > 1, at most 8) must give every rank whole KV heads and whole
 * rows, and every row interval that is joined across ranks — n_head*head_dim/G,
 * n_embd/G, n_ff/G and n_vocab/G f32 values — must be a multiple of 4 values
 * (joins move 16-byte units).  emelb_llama_create applies it first. */
EMELB_API uint32_t emelb_llama_check_config(const emelb_llama_config* cfg);

/* allocates activations, the f16 KV cache in the flash layout
 * [layer][kv_head][capacity][head_dim]
 * (src/emel/text/generator/detail.hpp:3010-3048) and the RoPE table */
EMELB_API uint32_t emelb_llama_create(emelb_ctx* ctx, const emelb_llama_config* cfg,
                                      emelb_llama** out);
EMELB_API uint32_t emelb_llama_destroy(emelb_llama* s);

/* binds one tensor (replaces bind_tensor_rows / make_src_view,
 * src/emel/text/generator/detail.hpp:788-817, 1886-1919): a {K, M} view of
 * native blocks (matrices) or f32 (norm vectors) whose data is a device
 * pointer or a host pointer inside a resident span */
EMELB_API uint32_t emelb_llama_bind(emelb_llama* s, int32_t layer, int32_t role,
                                    const emelb_view* tensor);

/* one decode step at `position` (replaces run_decode).  logits_out (n_vocab
 * f32, host or device) and token_out (greedy argmax, lowest id on ties) may
 * each be null; with logits_out null the logits are never materialised
 * (op_mul_mat_argmax route, src/emel/text/generator/detail.hpp:4035-4060). */
EMELB_API uint32_t emelb_llama_decode(emelb_llama* s, int32_t token, int32_t position,
                                      float* logits_out, int32_t* token_out);

/* feeds `n` prompt tokens at positions start_pos.. without computing logits:
 * fills their KV rows.  The reference's x86 prefill walks the prompt one token
 * at a time (src/emel/text/generator/detail.hpp:4064-4092).  With the fast
 * attention (mode 0) the prompt is processed in batches of up to 2048 tokens
 * (emelb_llama_set_prefill_batch) instead: per token the same arithmetic except the attention, which is an f32
 * online softmax over the batch (emelb_flash_attn_batch).  Sharded sessions do
 * the same when their context has a communicator (emelb_comm_init), joining the
 * ranks' row intervals of every product by all-gather.  The reference-order
 * attention modes walk token by token. */
EMELB_API uint32_t emelb_llama_prefill(emelb_llama* s, const int32_t* tokens, int32_t n,
                                       int32_t start_pos);

/* prompt tokens per batch of emelb_llama_prefill: default 2048; 0 or 1 walks the
 * prompt token by token (what the reference does); the first batched prompt sizes
 * the session's batch buffers, later values are clamped to them */
EMELB_API uint32_t emelb_llama_set_prefill_batch(emelb_llama* s, int32_t max_tokens);

/* greedy generation of `n` tokens with the token fed back on the device: no
 * host round trip between steps; tokens_out (host) is written at the end */
EMELB_API uint32_t emelb_llama_generate(emelb_llama* s, int32_t first_token,
                                        int32_t start_pos, int32_t n, int32_t* tokens_out);

/* Row-sharded sessions on one node: the joins of the ranks' row intervals can run as
 * peer stores over NVLink instead of NCCL all-gathers (one small kernel per join).
 * Each rank exports a handle of its exchange arena (the joined vectors live in it),
 * the caller all-gathers the G handles, and each rank attaches them (rank order,
 * G x EMELB_EXCHANGE_HANDLE_BYTES).  Attach on every rank and synchronise the ranks
 * before the first step (a join waits at most 10 s for a peer, then the step fails with
 * EMELB_INTERNAL_ERROR at the next emelb_sync);
 * without it the session keeps using the context's NCCL communicator.  No reference
 * counterpart beyond the lane join of src/emel/kernel/matmul/actions.hpp:108-136. */
#define EMELB_EXCHANGE_HANDLE_BYTES 64
EMELB_API uint32_t emelb_llama_exchange_export(emelb_llama* s, uint8_t* handle_out,
                                               uint64_t handle_bytes);
EMELB_API uint32_t emelb_llama_exchange_attach(emelb_llama* s, const uint8_t* handles,
                                               uint64_t handles_bytes);
/* unmaps the peers' arenas (the session falls back to NCCL joins).  Tear-down order
 * across ranks: every rank detaches, the caller synchronises the ranks, then the
 * sessions are destroyed — no arena is freed while a peer still maps it. */
EMELB_API uint32_t emelb_llama_exchange_detach(emelb_llama* s);

/* ---- several sequences decoded together (batch decode).  A session holds n_seq KV caches (default 1;
 * emelb_llama_set_sequences reallocates and clears them).  The one-sequence entry points above (prefill, decode,
 * generate) work on the sequence chosen by emelb_llama_select_sequence (default 0), so a caller fills each
 * sequence's cache with its prompt and then steps all of them together:
 *   decode_batch   one step: sequence j (0 <= j < n_seq) takes tokens[j] at positions[j]; logits_out (optional,
 *                  host, {n_vocab, n_seq} with the sequence index fastest -- op_mul_mat's result layout) and
 *                  tokens_out (optional, host, the greedy next id per sequence);
 *   generate_batch n_steps greedy steps fed back on the device, one CUDA-graph replay per step;
 *                  tokens_out[step * n_seq + j].
 * Column j of every product is computed with the arithmetic of the one-sequence step (same block order, same
 * rotation, split-KV attention with the same split count), so each sequence gets exactly the tokens and logits
 * it gets when decoded alone.  Needs attention mode 0; EMELB_UNSUPPORTED_OP otherwise.  The reference's generator
 * decodes one sequence per session (src/emel/text/generator/detail.hpp:4860-4914); this is that loop over
 * several sessions' worth of state with the weights streamed once per step. */
EMELB_API uint32_t emelb_llama_set_sequences(emelb_llama* s, int32_t n_seq);
EMELB_API uint32_t emelb_llama_select_sequence(emelb_llama* s, int32_t seq);
EMELB_API uint32_t emelb_llama_decode_batch(emelb_llama* s, const int32_t* tokens, const int32_t* positions, int32_t n_seq,
                                            float* logits_out, int32_t* tokens_out);
EMELB_API uint32_t emelb_llama_generate_batch(emelb_llama* s, const int32_t* first_tokens, const int32_t* start_positions,
                                              int32_t n_seq, int32_t n_steps, int32_t* tokens_out);
EMELB_API uint32_t emelb_llama_batch_launches_per_step(const emelb_llama* s, int32_t* out);

/* Row-sharded sessions with every peer attached: where a layer's products all take the streaming kernel, its four
 * joins run inside the kernels either side of them -- the producing kernel (attention merge, output projection,
 * SwiGLU, down projection) stores its rows into every rank's copy of the vector and raises a flag, the consuming
 * product waits for the flags and quantizes the joined f32 vector in its prologue -- instead of one join kernel
 * each.  on = 0 (default): one join kernel per join; on = 1: inside the neighbouring kernels (232 instead of 423
 * launches per token at the 8B shape; measured no faster on 2 GPUs and slower on 4, hence not the default).  Same
 * result bit for bit either way. */
EMELB_API uint32_t emelb_llama_set_join_fusion(emelb_llama* s, int32_t on);

/* Layers streamed from host memory (models whose layers do not fit the HBM left for weights).  `w` is a bound,
 * streaming emelb_window on the session's context with one layer descriptor per model layer.  After this call
 * emelb_llama_bind accepts, for a layer tensor, a view whose `data` is not resident but is the address of one of that
 * layer's extents inside the window's source (same byte size): the tensor is then read from the slot the window
 * hands out for the layer.  Resident and streamed tensors may be mixed.  Each layer pass of a step, of a prompt batch
 * and of a batch step acquires its layer once, so the next layers cross PCIe while the current one computes; steps
 * run as plain launches instead of replayed graphs.  Same results bit for bit as the resident session.  Unsharded
 * sessions only.  The window must stay bound while tensors of the session are bound through it; w = null detaches
 * (refused while streamed tensors are bound). */
EMELB_API uint32_t emelb_llama_set_window(emelb_llama* s, emelb_window* w);

/* How a decode step is enqueued.  0 (default): the chain of per-operation
 * launches.  1: where the session qualifies (unsharded, Q4_K layer matrices with
 * K a multiple of 2048, head size 128, adjacent-pair RoPE, fast attention mode),
 * all layers of a token run as ONE persistent kernel, one CTA per SM, with grid
 * barriers between the phases of a layer and producer warps that keep the
 * weights streaming across them; sessions that do not qualify keep the chain.
 * Both give the same numbers bit for bit.  No reference counterpart (its
 * generator calls the kernel actor once per operation,
 * src/emel/text/generator/detail.hpp:3746-3926). */
EMELB_API uint32_t emelb_llama_set_step_mode(emelb_llama* s, int32_t mode);

/* Phase profile of the one-kernel step (diagnostics, like the reference's
 * capture_diagnostics counters): runs the layers of one decode step at
 * (token, position) — the KV row of `position` is written as in a normal step,
 * no logits are produced — and returns, for each layer, 16 nanosecond stamps
 * taken by one CTA: 0 layer start, 1 Q/K/V input staged, 2 Q/K/V products done,
 * 3/5/8/11/14 after the grid barriers, 4 attention done, 6 output-projection
 * input staged, 7 output projection done, 9 gate/up input staged, 10 gate/up
 * done, 12 SwiGLU staged, 13 down projection done.  stamps_count >= 16 * n_layer.
 * EMELB_UNSUPPORTED_OP when the session does not qualify for the one-kernel step. */
EMELB_API uint32_t emelb_llama_decode_profile(emelb_llama* s, int32_t token, int32_t position,
                                              uint64_t* stamps_ns, uint64_t stamps_count);

/* kernels launched per decode step (for launch accounting) */
EMELB_API uint32_t emelb_llama_launches_per_token(const emelb_llama* s, int32_t* out);

#ifdef __cplusplus
}
#endif
#endif /* EMELB_LLAMA_H */
