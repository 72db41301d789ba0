/*
 * emelb.h — C-ABI of the B200 (sm_100a) CUDA backend for EMEL's quantized
 * matrix-product path.
 *
 * EMEL has no C plugin ABI of its own (include/emel/emel.h:1-18 only declares
 * emel_error_type); the seam this library sits behind is the C++ kernel-event
 * surface `bool emel::kernel::any::process_event(const event::op_X&)`
 * (src/emel/kernel/any.hpp:76-80).  Every entry point below names the
 * reference interface it replaces.  A `kernel::cuda::sm` actor forwards its
 * op events to these calls one-to-one (see emel.cpp_b200/cuda_sm.hpp).
 *
 * Conventions
 *  - Every call returns the reference's kernel error bitmask
 *    (src/emel/kernel/errors.hpp:7-13).  Nothing throws or aborts.
 *  - Views are borrowed for the duration of the call.
 *  - A view's `data` pointer may be: a device pointer; a host pointer inside
 *    a span registered with emelb_residency_upload (weights: the device copy
 *    is used, no transfer); or any other host pointer (activations/results:
 *    copied through the context's device staging area inside the call, which
 *    returns after the result is back in host memory).  The pointer kind is looked up (residency
 *    table, then the CUDA driver's pointer attributes), never guessed.
 *  - One context per caller thread/lane; a context is not re-entrant
 *    (same rule as one kernel actor per lane,
 *    src/emel/kernel/matmul/context.hpp:16-24).
 *  - With device-resident operands a call only enqueues work on the context's
 *    stream; emelb_sync waits for it.
 */
#ifndef EMELB_H
#define EMELB_H

#include <stdint.h>

#if defined(__GNUC__)
#define EMELB_API __attribute__((visibility("default")))
#else
#define EMELB_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

/* src/emel/kernel/errors.hpp:7-13 */
enum {
  EMELB_OK = 0u,
  EMELB_INVALID_REQUEST = 1u << 0,
  EMELB_UNSUPPORTED_OP = 1u << 1,
  EMELB_INTERNAL_ERROR = 1u << 2,
  EMELB_UNTRACKED = 1u << 3
};

/* dtype codes: src/emel/kernel/events.hpp:78-123 (ggml's numbering). */
enum {
  EMELB_F32 = 0,
  EMELB_F16 = 1,
  EMELB_Q4_0 = 2,
  EMELB_Q8_0 = 8,
  EMELB_Q4_K = 12,
  EMELB_Q6_K = 14,
  EMELB_Q8_K = 15,
  EMELB_I32 = 26,
  EMELB_UNKNOWN = 255
};

/* tensor_view / tensor_view_mut: src/emel/kernel/events.hpp:125-137.
 * ne[0] is the fastest dimension, nb[i] the byte stride of dimension i. */
typedef struct emelb_view {
  const void* data;
  uint8_t type;
  uint64_t ne[4];
  uint64_t nb[4];
} emelb_view;

/* EMEL_KERNEL_GENERIC_OP_FIELDS + op_mul_mat_argmax::index_out:
 * src/emel/kernel/events.hpp:178-189, 220-223. `dst.data` is written. */
typedef struct emelb_op {
  emelb_view src0;
  emelb_view src1;
  emelb_view src2;
  emelb_view dst;
  uint8_t op_params[64];
  uint32_t op_params_size;
  int32_t* index_out;
} emelb_op;

/* op codes for emelb_can_run */
enum {
  EMELB_OP_MUL_MAT = 1,
  EMELB_OP_MUL_MAT_ARGMAX = 2,
  EMELB_OP_FLASH_ATTN_EXT = 3,
  EMELB_OP_RMS_NORM = 4,
  EMELB_OP_ROPE = 5,
  EMELB_OP_GLU = 6
};

/* lifecycle: src/emel/model/tensor/events.hpp:18-24 */
enum {
  EMELB_LIFECYCLE_UNBOUND = 0,
  EMELB_LIFECYCLE_RESIDENT = 1,
  EMELB_LIFECYCLE_EVICTED = 2,
  EMELB_LIFECYCLE_INTERNAL_ERROR = 3,
  EMELB_LIFECYCLE_MMAP_RESIDENT = 4
};

/* tensor_state: src/emel/model/tensor/events.hpp:26-34; `buffer` is the
 * device address of the uploaded bytes, `host` the span it mirrors. */
typedef struct emelb_tensor_state {
  uint8_t lifecycle_state;
  const void* buffer;
  uint64_t buffer_bytes;
  const void* host;
  int32_t tensor_type;
} emelb_tensor_state;

/* Dispatch counters; names follow event::diagnostics
 * (src/emel/kernel/events.hpp:39-62). */
typedef struct emelb_diag {
  uint64_t optimized_flash_dispatch_calls;
  uint64_t shared_flash_dispatch_calls;
  uint64_t optimized_q4_dispatch_calls;
  uint64_t optimized_q4_vector_dispatch_calls;
  uint64_t optimized_q6_dispatch_calls;
  uint64_t optimized_q6_vector_dispatch_calls;
  uint64_t optimized_q6_vector_argmax_dispatch_calls;
  uint64_t optimized_q8_0_dispatch_calls;
  uint64_t optimized_q4_0_dispatch_calls;
  uint64_t rejected_dispatch_calls;
  uint64_t kernel_launches;      /* CUDA kernels launched by this context */
  uint64_t h2d_bytes;            /* staged host->device bytes */
  uint64_t d2h_bytes;            /* staged device->host bytes */
} emelb_diag;

typedef struct emelb_ctx emelb_ctx;

/* ---- context: replaces constructing one kernel actor
 * (src/emel/kernel/x86_64/context.hpp:214-243). Allocates the persistent
 * workspace (activation scratch, attention partials, device staging); no
 * allocation happens in any dispatch call afterwards. ---- */
EMELB_API uint32_t emelb_create(int device, emelb_ctx** out);
EMELB_API uint32_t emelb_destroy(emelb_ctx* ctx);
/* waits for the context's stream; EMELB_INTERNAL_ERROR on a CUDA error */
EMELB_API uint32_t emelb_sync(emelb_ctx* ctx);
/* the cudaStream_t all work of this context is enqueued on */
EMELB_API uint32_t emelb_get_stream(emelb_ctx* ctx, void** stream_out);
/* event::capture_diagnostics: src/emel/kernel/any.hpp:38-74 */
EMELB_API uint32_t emelb_diagnostics(const emelb_ctx* ctx, emelb_diag* out);
/* attention numerics: 0 = split-KV f32 accumulators (fast, default);
 * 1 = reference order, scalar route: sequential over tokens with an f16-rounded
 * accumulator, f64 score sums (src/emel/kernel/detail.hpp:5238-5291);
 * 2 = reference order, x86 AVX2 route: same accumulator, scores summed as the
 * AVX2/FMA kernel does (src/emel/kernel/x86_64/actions.hpp:1388-1446, 1575-1641).
 * Shapes the split-KV kernel does not take run in order 2 under mode 0. */
EMELB_API uint32_t emelb_set_attention_mode(emelb_ctx* ctx, int mode);

/* ---- residency: replaces io::loader strategy `external_buffer`
 * (src/emel/io/loader/events.hpp:25-31, rejected as unsupported at
 * src/emel/io/loader/sm.hpp:78-81) and model::tensor lifecycle/state
 * (src/emel/model/tensor/events.hpp:18-34, 85-89). Bytes are uploaded
 * unchanged; `host` stays the key a later view may carry. ---- */
EMELB_API uint32_t emelb_residency_upload(emelb_ctx* ctx, int32_t tensor_id,
                                const void* host, uint64_t bytes,
                                int32_t tensor_type, const void** dev_out);
EMELB_API uint32_t emelb_residency_evict(emelb_ctx* ctx, int32_t tensor_id);
/* how host spans outside page-locked memory reach the device (no reference
 * counterpart: its loader strategies end at host memory,
 * src/emel/io/loader/events.hpp:25-31).  RING (default): 4 MB chunks through a
 * page-locked staging ring fed by `threads` host threads (0 = one per core, at
 * most 16; pread-fed when the span maps a file).  PLAIN: one pageable copy per
 * span.  REGISTER: the span is page-locked in place (read-only) and copied
 * without a host copy. */
enum { EMELB_UPLOAD_RING = 0, EMELB_UPLOAD_PLAIN = 1, EMELB_UPLOAD_REGISTER = 2 };
EMELB_API uint32_t emelb_set_upload_route(emelb_ctx* ctx, int32_t route, int32_t threads);

EMELB_API uint32_t emelb_residency_state(const emelb_ctx* ctx, int32_t tensor_id,
                               emelb_tensor_state* out);

/* plain device buffers for activations / KV cache owned by the caller */
EMELB_API uint32_t emelb_device_alloc(emelb_ctx* ctx, uint64_t bytes, void** dev_out);
EMELB_API uint32_t emelb_device_free(emelb_ctx* ctx, void* dev);
EMELB_API uint32_t emelb_copy_to_device(emelb_ctx* ctx, void* dev, const void* host,
                              uint64_t bytes);
EMELB_API uint32_t emelb_copy_to_host(emelb_ctx* ctx, void* host, const void* dev,
                            uint64_t bytes);

/* ---- guards: replaces can_run_mul_mat / can_run_mul_mat_argmax /
 * can_run_flash_attn_ext + validate_dispatch_request
 * (src/emel/kernel/detail.hpp:3843-3872, 3573-3606, 4346-4390, 1919-1927).
 * Pure: returns EMELB_OK or EMELB_INVALID_REQUEST, launches nothing. ---- */
EMELB_API uint32_t emelb_can_run(const emelb_ctx* ctx, uint32_t op_code,
                       const emelb_op* op);

/* ---- op_mul_mat: replaces x86_64::sm.process_event(op_mul_mat)
 * (src/emel/kernel/x86_64/sm.hpp:355-423) i.e. run_mul_mat
 * (src/emel/kernel/detail.hpp:3356-3571) and the AVX2 drivers
 * (src/emel/kernel/x86_64/actions.hpp:1186-1326).
 * src0 = {K, M} Q4_K|Q6_K|Q8_0|Q4_0 rows; src1 = {N, K} f32 (token fastest),
 * or the pre-quantized vector form {1, K} of type Q8_K / Q8_0
 * (src/emel/kernel/aarch64/actions.hpp:1471-1503); dst = {N, M} f32. ---- */
EMELB_API uint32_t emelb_mul_mat(emelb_ctx* ctx, const emelb_op* op);

/* ---- quantize once, multiply many: replaces the q8 route of the reference's
 * callers, quantize_vector_q8_k + matmul_vector_q8_input (one quantized input
 * feeds Q, K and V, or gate and up:
 * src/emel/text/generator/detail.hpp:3780-3793, 3885-3899).
 * emelb_prepare_rhs quantizes src1 (f32 {N, K}) for a weight type's family
 * (Q8_K for K-quants, Q8_0 for 32-blocks) into the context's activation
 * planes; emelb_mul_mat_prepared then runs op_mul_mat against those planes,
 * launching only the matrix kernel.  op->src1 must describe the same {N, K}
 * f32 tensor (its data pointer is not read).  Any other dispatch on the context
 * invalidates the prepared planes. ---- */
EMELB_API uint32_t emelb_prepare_rhs(emelb_ctx* ctx, const emelb_view* src1_f32,
                                     int32_t weight_type);
EMELB_API uint32_t emelb_mul_mat_prepared(emelb_ctx* ctx, const emelb_op* op);
/* `count` products against the same prepared column, results as `count` calls of
 * emelb_mul_mat_prepared.  Two or three matrices of one type and row length with
 * device outputs (Q, K, V or gate, up of one layer) run as ONE launch of the
 * streaming mat-vec kernel, the way the decoder session issues them. */
EMELB_API uint32_t emelb_mul_mat_prepared_group(emelb_ctx* ctx, const emelb_op* ops,
                                                uint32_t count);

/* ---- op_mul_mat_argmax: replaces run_mul_mat_argmax
 * (src/emel/kernel/detail.hpp:3608-3731): dst[0] = best value,
 * *index_out = lowest row attaining it. ---- */
EMELB_API uint32_t emelb_mul_mat_argmax(emelb_ctx* ctx, const emelb_op* op);

/* ---- op_flash_attn_ext: replaces
 * run_flash_attn_ext_active_kv_with_workspace
 * (src/emel/kernel/detail.hpp:5238-5300) and the AVX2 one-chunk route
 * (src/emel/kernel/x86_64/actions.hpp:1575-1641). ---- */
EMELB_API uint32_t emelb_flash_attn_ext(emelb_ctx* ctx, const emelb_op* op);

/* ---- op_rms_norm: replaces run_rms_norm (src/emel/kernel/detail.hpp:4567-4602;
 * event src/emel/kernel/events.hpp:215): src0 and dst f32 of the same shape, any
 * valid byte strides; per row out = x / sqrt(mean(x^2) + eps) with the f64 sum of
 * the f32 squares; op_params = {f32 eps >= 0}.  (The weight multiply of the
 * decoder's rms_norm is the generator's, not this op's.) ---- */
EMELB_API uint32_t emelb_rms_norm(emelb_ctx* ctx, const emelb_op* op);

/* ---- op_rope: replaces run_rope_as (src/emel/kernel/detail.hpp:4650-4765; event
 * src/emel/kernel/events.hpp:242): src0/dst f32 {dims, heads, tokens, batch}, src1
 * i32 positions {tokens}, op_params in ggml's layout (i32 slots 1 = n_dims,
 * 2 = mode; f32 slots 5..8 = freq_base, freq_scale, ext_factor (must be 0),
 * attn_factor).  mode 0 rotates adjacent pairs, mode 2 the half-split pairs; the
 * angle recurrence (theta *= powf(freq_base, -2/n_dims), host libm) is the
 * reference's float for float, cos/sin come from the device library (last-place
 * differences).  Mode 4 (the timestep-embedding variant) returns
 * EMELB_UNSUPPORTED_OP. ---- */
EMELB_API uint32_t emelb_rope(emelb_ctx* ctx, const emelb_op* op);

/* ---- op_glu (src/emel/kernel/events.hpp:307-310): the reference's kernel actors
 * reject every op_glu request (no branch of can_execute_scalar takes it,
 * src/emel/kernel/detail.hpp:5166-5203), and so does this backend:
 * EMELB_INVALID_REQUEST.  The decoder layer's SwiGLU lives in emelb_llama. ---- */
EMELB_API uint32_t emelb_glu(emelb_ctx* ctx, const emelb_op* op);

/* ---- kernel::attention's head-range event (src/emel/kernel/attention/events.hpp:18-31; the work is
 * effect_execute_head_range, src/emel/kernel/attention/actions.hpp:15-96): attention of one query token over a
 * bf16 KV ring buffer laid out [position][hidden_dim] per layer, for heads head_begin .. head_end-1 (no grouped
 * heads: head h reads columns h*head_dim.. of both caches).  Per head: the query is rounded to bf16; the score of
 * logical position p (physical row (physical_begin + p) mod position_capacity) is the f64 sum, in element order, of
 * the f32 products k*q, rounded to f32 and multiplied by 1/sqrt(head_dim); rows outside the valid positions score
 * -inf; a softmax over all position_capacity rows (max, expf, f64 sum in row order, weights times (float)(1/sum));
 * the weights are rounded to bf16; and the output is the f64 sum over the valid positions, in logical order, of the
 * f32 products v*weight, rounded to f32.  The arithmetic follows the reference's scalar route (its build without a
 * global -mavx2: the oracle's build definition) bit for bit.
 * Counts are element counts of the spans (request validation mirrors guard_request_shape_supported,
 * src/emel/kernel/attention/guards.hpp:28-90, including the limits head_dim, position_capacity <= 8192 and the
 * requirement that the output span overlaps none of the inputs).  Pointers may be host or device memory. ---- */
typedef struct emelb_head_range_request {
  const float* query;            /* hidden_dim floats */
  uint64_t query_count;
  const uint16_t* key_cache;     /* bf16 bits */
  uint64_t key_count;
  const uint16_t* value_cache;
  uint64_t value_count;
  float* output;                 /* (head_end - head_begin) * head_dim floats */
  uint64_t output_count;
  uint64_t layer_offset;         /* elements before this layer's rows in both caches */
  int32_t hidden_dim, head_dim, head_begin, head_end, position_capacity, physical_begin, valid_positions;
} emelb_head_range_request;
/* pure guard: EMELB_OK or EMELB_INVALID_REQUEST */
EMELB_API uint32_t emelb_attention_head_range_can_run(const emelb_head_range_request* request);
EMELB_API uint32_t emelb_attention_head_range(emelb_ctx* ctx, const emelb_head_range_request* request);

/* ---- the same attention for a batch of prompt tokens: query token j (of `batch`)
 * sits at position pos0 + j and attends to cache positions 0 .. pos0 + j.  The
 * reference walks a prompt through op_flash_attn_ext one token at a time
 * (src/emel/text/generator/detail.hpp:3232-3279); here one launch covers the
 * batch.  All pointers are device memory: q and dst are f32 {heads * head_dim,
 * batch} with the token index fastest (op_mul_mat's result layout), k and v the
 * f16 cache [kv_head][position][head_dim] with cache_head_stride halves between
 * kv heads, holding positions 0 .. pos0 + batch - 1.  f32 online softmax
 * (within 2e-5 of the exact softmax); head_dim 64 or 128, heads / kv_heads a
 * divisor of 64, else EMELB_UNSUPPORTED_OP. ---- */
EMELB_API uint32_t emelb_flash_attn_batch(emelb_ctx* ctx, const float* q, const void* k,
                                          const void* v, float* dst, int32_t head_dim,
                                          int32_t heads, int32_t kv_heads, int32_t batch,
                                          int32_t pos0, int64_t cache_head_stride, float scale);

/* ---- activation quantizers: replace quantize_row_q8_k_strided /
 * quantize_row_q8_0_strided (src/emel/kernel/detail.hpp:826-867, 804-824).
 * src = f32 {N, K} (token fastest, as op_mul_mat's src1); dst type selects
 * Q8_K or Q8_0; dst holds N rows of K/256 (K/32) reference-layout blocks,
 * row j = column j of src.  Bit-exact. ---- */
EMELB_API uint32_t emelb_quantize(emelb_ctx* ctx, const emelb_view* src_f32,
                        const emelb_view* dst);

/* ---- block dequantizers: replace dequantize_row_q4_k / q6_k / q8_0 / q4_0
 * (src/emel/kernel/detail.hpp:523-552, 592-629, 679-690, 487-502).
 * src = {K, M} quantized rows, dst = {K, M} f32.  Bit-exact. ---- */
EMELB_API uint32_t emelb_dequantize(emelb_ctx* ctx, const emelb_view* src,
                          const emelb_view* dst_f32);

/* ---- row-slice helper: replaces compute_sliced_mul_mat_event +
 * compute_fixed_row_slice (src/emel/kernel/matmul/detail.hpp:36-54,
 * src/emel/kernel/matmul/actions.hpp:48-67). Pure host arithmetic:
 * writes lane `lane` of `lane_count`'s slice of `op` to `out`. ---- */
EMELB_API uint32_t emelb_row_slice(const emelb_op* op, uint32_t lane,
                         uint32_t lane_count, emelb_op* out,
                         uint64_t* row_begin, uint64_t* row_count);

/* ---- the join of the row-sliced path across GPUs.  The reference forks one
 * op_mul_mat into lane_count disjoint dst-row intervals with a shared RHS and
 * joins them in host memory (effect_execute_parallel,
 * src/emel/kernel/matmul/actions.hpp:49-136; lane-count invariance
 * docs/determinism.md:29-32).  With one process per GPU, lane = rank: each rank
 * runs emelb_mul_mat on its emelb_row_slice and emelb_all_gather_rows joins the
 * intervals.  dst_dev is the FULL result (rows_per_rank * world rows of
 * row_floats f32, device memory); the caller's own interval is already in place
 * at row rank*rows_per_rank.  Stream-ordered; every rank must call it with the
 * same sizes.  Without a communicator (world 1) it is a no-op.
 * emelb_comm_unique_id (rank 0) -> the caller broadcasts the id -> every rank
 * calls emelb_comm_init once per context. ---- */
#define EMELB_COMM_ID_BYTES 128
EMELB_API uint32_t emelb_comm_unique_id(uint8_t* id_out, uint64_t id_bytes);
EMELB_API uint32_t emelb_comm_init(emelb_ctx* ctx, int32_t rank, int32_t world,
                         const uint8_t* id, uint64_t id_bytes);
EMELB_API uint32_t emelb_comm_destroy(emelb_ctx* ctx);
/* how long a peer-store join waits on the device for the other ranks' flags
 * before the kernel gives up, raises the context's status word and returns
 * (default 10 s; the next emelb_sync then reports EMELB_INTERNAL_ERROR and the
 * context stays usable).  Every device-side wait of the library is bounded this
 * way; no reference counterpart (its lane join spins on the host,
 * src/emel/kernel/matmul/actions.hpp:108-136). */
EMELB_API uint32_t emelb_set_peer_wait_ms(emelb_ctx* ctx, uint32_t limit_ms);
/* diagnostics: enqueues a two-rank peer-store join whose second rank never
 * answers (both ranks' buffers are this context's own staging memory, so no
 * second GPU is involved and nothing faults): the kernel's wait runs out after
 * limit_ms (1..10000) and the status word is raised.  Exercises the path from a
 * device-side timeout to emelb_sync's EMELB_INTERNAL_ERROR. */
EMELB_API uint32_t emelb_selftest_wait_timeout(emelb_ctx* ctx, uint32_t limit_ms);
EMELB_API uint32_t emelb_all_gather_rows(emelb_ctx* ctx, float* dst_dev,
                         uint64_t rows_per_rank, uint64_t row_floats);

/* ---- stream capture (no reference counterpart: the reference dispatches
 * synchronously on the calling thread).  Between begin and end, calls whose
 * operands are all device-resident are recorded instead of run; the resulting
 * graph replays them with one launch.  Calls that would touch host memory
 * (staged copies, argmax results written to host pointers) must not be made
 * while capturing. ---- */
EMELB_API uint32_t emelb_graph_begin(emelb_ctx* ctx);
EMELB_API uint32_t emelb_graph_end(emelb_ctx* ctx, void** graph_out);
EMELB_API uint32_t emelb_graph_launch(emelb_ctx* ctx, void* graph);
EMELB_API uint32_t emelb_graph_destroy(emelb_ctx* ctx, void* graph);

/* ---- mat-vec for callers that cannot allocate.  No counterpart in the
 * reference (its CPU kernels keep their scratch on the stack).  Computes
 * y[m] = W{K, M} * x[K] like emelb_mul_mat with N = 1, for device-resident
 * operands, without a context and without allocating anything: the quantized
 * activations and the kernel's task counter live in a fixed array inside the
 * library image (about 40 KB per GPU, held until the process exits).  For
 * callers such as latency-bound serving loops or hooks where cudaMalloc is not
 * permitted.  K <= 32768; larger K is refused with EMELB_INVALID_REQUEST and a
 * message in error_text (optional buffer).  Calls on one device share the array:
 * do not let two of them overlap on the GPU.  The first call on a device does a
 * one-time address look-up; make it outside any stream capture.  `stream` is
 * the cudaStream_t to enqueue on (NULL = default stream).  The calling thread's
 * current device is left as it was.  Having no context, the call cannot report
 * a copy wait that ran out inside the kernel (emelb_sync does that for the
 * context-based calls): use it where a lost device is detected by other means. ---- */
EMELB_API uint32_t emelb_mul_mat_vec_noalloc(int device, void* stream,
                                             int32_t weight_type,
                                             const void* weights_dev, uint64_t k,
                                             uint64_t m, const float* x_dev,
                                             float* y_dev, char* error_text,
                                             uint64_t error_text_bytes);

/* ---- synthetic data (no reference counterpart; the reference's benches fill
 * buffers with closed-form patterns on the host,
 * tools/bench/text/generator/parallel_matmul_bench.cpp:177-238).  Fills `dev`
 * with `elems` values drawn N(0, sigma) from (seed, offset): as f32, or encoded
 * on the device into Q4_K / Q6_K / Q8_0 / Q4_0 blocks by this project's own
 * encoders.  Benchmark-sized models (tens of GB) are built this way. ---- */
EMELB_API uint32_t emelb_synth_fill(emelb_ctx* ctx, void* dev, int32_t type,
                                    uint64_t elems, uint64_t seed, float sigma,
                                    uint64_t offset);

#ifdef __cplusplus
}
#endif
#endif /* EMELB_H */
