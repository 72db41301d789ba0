/*
 * emelb_window.h — the layer streaming window with its slots in HBM.
 *
 * The reference's model::tensor::window actor keeps a model that does not fit a
 * memory budget on its source (a file mapping) and cycles the layers' weights
 * through a ring of slots, loading ahead of the layer that is being computed
 * (src/emel/model/tensor/window/events.hpp:26-70, detail.hpp:17-195,
 * guards.hpp:13-186 and 296-470, actions.hpp:218-227 and 394-406).  Here the
 * slots are device memory and the source is host memory: the ring is the way
 * to decode a model that is larger than the HBM left for weights, one layer's
 * weights crossing PCIe while the previous layer computes.
 *
 * Same requests, same plan arithmetic (64-byte aligned extents packed per
 * layer, slot of layer l = l % window_slots), same decisions in the same order
 * and the same error bits (src/emel/model/tensor/window/errors.hpp:9-21).
 * What differs is what a slot load is:
 *   - the window first tries to page-lock the source read-only; loads are then
 *     asynchronous copies on a stream of the window, ordered against the
 *     compute stream by events only (the host never waits);
 *   - where the source cannot be page-locked, one I/O thread copies chunk by
 *     chunk (stage_chunk_bytes) through two page-locked buffers, and an acquire
 *     of a layer whose load is still running waits for it on the host.
 * A slot view handed out by emelb_window_acquire is valid for work enqueued on
 * the context's stream until the next acquire on the same window; the window
 * does not overwrite the slot before that work has run.
 */
#ifndef EMELB_WINDOW_H
#define EMELB_WINDOW_H

#include "emelb.h"

#ifdef __cplusplus
extern "C" {
#endif

/* src/emel/model/tensor/window/errors.hpp:9-21 */
enum {
  EMELB_WINDOW_OK = 0u,
  EMELB_WINDOW_INVALID_REQUEST = 1u << 0,
  EMELB_WINDOW_NOT_BOUND = 1u << 1,
  EMELB_WINDOW_ALREADY_BOUND = 1u << 2,
  EMELB_WINDOW_SOURCE_MAP_FAILED = 1u << 3,
  EMELB_WINDOW_BUDGET_TOO_SMALL = 1u << 4,
  EMELB_WINDOW_LAYER_OUT_OF_RANGE = 1u << 5,
  EMELB_WINDOW_SLOT_COPY_FAILED = 1u << 6,
  EMELB_WINDOW_NOT_STREAMING = 1u << 7,
  EMELB_WINDOW_INTERNAL_ERROR = 1u << 8,
  EMELB_WINDOW_SLOT_STORAGE_TOO_SMALL = 1u << 9
};

/* src/emel/model/tensor/window/detail.hpp:17-25 */
#define EMELB_WINDOW_MAX_SLOTS 8u
#define EMELB_WINDOW_MAX_LAYERS 160u
#define EMELB_WINDOW_MAX_WEIGHTS_PER_LAYER 12u
#define EMELB_WINDOW_MIN_CHUNK_BYTES (1ull << 20)
#define EMELB_WINDOW_DEFAULT_CHUNK_BYTES (8ull << 20)
#define EMELB_WINDOW_MAX_CHUNK_BYTES (16ull << 20)
#define EMELB_WINDOW_SLOT_ALIGNMENT 64u

/* weight_extent, src/emel/model/tensor/window/detail.hpp:32-37: one contiguous
 * span of the source, placed at slot_offset inside its layer's slot.  Callers
 * fill tensor_id, file_offset and byte_size; slot_offset is computed by bind. */
typedef struct emelb_window_extent {
  int32_t tensor_id;
  uint64_t file_offset;
  uint64_t byte_size;
  uint64_t slot_offset;
} emelb_window_extent;

/* layer_descriptor, src/emel/model/tensor/window/detail.hpp:39-45 */
typedef struct emelb_window_layer {
  emelb_window_extent weights[EMELB_WINDOW_MAX_WEIGHTS_PER_LAYER];
  uint32_t weight_count;
  uint64_t file_begin;
  uint64_t file_span;
  uint64_t slot_bytes;
} emelb_window_layer;

/* bind_window_request, src/emel/model/tensor/window/events.hpp:36-49.
 * The source is either `source` (source_bytes of host memory that stay valid
 * and unchanged until unbind, e.g. the mapping a parsed GGUF image lives in)
 * or, when `source` is null, the file `file_path` names, which the window maps
 * read-only itself (file_size_bytes must be its size).  slot_storage is DEVICE
 * memory of the context's GPU, owned by the caller for the lifetime of the
 * bind. */
typedef struct emelb_window_request {
  const char* file_path;
  uint64_t file_size_bytes;
  const void* source;
  const emelb_window_extent* extents;
  uint64_t extent_count;
  const uint16_t* layer_weight_counts;
  uint64_t layer_count;
  uint64_t budget_bytes;
  void* slot_storage;
  uint64_t slot_storage_bytes;
  uint32_t window_slots;
  uint32_t prefetch_depth;
  uint64_t stage_chunk_bytes;
} emelb_window_request;

/* bind_window_done, src/emel/model/tensor/window/events.hpp:84-91 */
typedef struct emelb_window_bound {
  int32_t streaming_active;
  const void* source_base;
  uint64_t source_bytes;
  uint32_t window_slots;
  int32_t source_page_locked; /* 1: loads are stream-ordered copies; 0: the I/O thread stages them */
} emelb_window_bound;

typedef struct emelb_window emelb_window;

/* counters of a window since its bind */
typedef struct emelb_window_stats {
  uint64_t loads_submitted;
  uint64_t loads_failed;
  uint64_t bytes_copied;
  uint64_t acquires;
  uint64_t acquires_resident; /* the layer was in its slot (loaded or loading ahead) when asked for */
  uint64_t acquires_cold;     /* the load was only submitted by the acquire itself */
} emelb_window_stats;

/* An unbound window on a backend context (the actor in its initial state). */
EMELB_API uint32_t emelb_window_create(emelb_ctx* ctx, emelb_window** out);
/* Joins loads in flight, unbinds if bound, frees the window. */
EMELB_API uint32_t emelb_window_destroy(emelb_window* w);

/* event::bind_window.  Decisions, in the reference's order (guards.hpp:13-186):
 * already bound or a malformed request -> INVALID_REQUEST (rebinding reports
 * ALREADY_BOUND); the source cannot be mapped -> SOURCE_MAP_FAILED; the packed
 * layers fit budget_bytes, or budget_bytes == 0 -> bound as passthrough
 * (streaming_active 0, no slots: the caller keeps the model resident by
 * emelb_residency_upload); otherwise window_slots in [2, 8] and
 * 0 < prefetch_depth < window_slots or INVALID_REQUEST; window_slots x the
 * largest layer must fit budget_bytes or BUDGET_TOO_SMALL; slot_storage must
 * be non-null, 64-byte aligned device memory of at least that size or
 * SLOT_STORAGE_TOO_SMALL.  A streaming bind submits the loads of the first
 * prefetch_depth layers before it returns. */
EMELB_API uint32_t emelb_window_bind(emelb_window* w, const emelb_window_request* request, emelb_window_bound* out);

/* The request checks and decisions of emelb_window_bind without binding anything (no GPU needed): the same error
 * bits in the same order, except that the source is not opened (a missing file is only found by bind) and that
 * slot_storage is checked for presence, size and alignment only.  Also reports the slot capacity (the largest packed
 * layer) and the packed size of all layers, which is what a caller sizes slot_storage and the budget from. */
EMELB_API uint32_t emelb_window_check(const emelb_window_request* request, int32_t* streaming_active,
                                      uint64_t* slot_capacity_bytes, uint64_t* total_bytes);

/* event::acquire_layer_window: make layer `layer_index`'s weights readable by
 * work enqueued on the context's stream after this call, and advance the ring
 * (submit the load of layer (layer_index + prefetch_depth) % layer_count unless
 * its slot is the one just handed out, holds it already or is loading).
 * *slot_base (device) + layout->weights[i].slot_offset is weight i.  A failed
 * load is submitted once more before SLOT_COPY_FAILED is reported.  Errors:
 * NOT_BOUND, NOT_STREAMING (passthrough), LAYER_OUT_OF_RANGE. */
EMELB_API uint32_t emelb_window_acquire(emelb_window* w, int32_t layer_index, const uint8_t** slot_base,
                                        const emelb_window_layer** layout);

/* event::unbind_window: joins loads in flight and the context's stream (work
 * that reads a slot has run when this returns), releases the source. */
EMELB_API uint32_t emelb_window_unbind(emelb_window* w);

EMELB_API uint32_t emelb_window_get_stats(const emelb_window* w, emelb_window_stats* out);
/* The plan of a bound window: layer descriptors with the computed slot offsets. */
EMELB_API uint32_t emelb_window_layer_plan(const emelb_window* w, int32_t layer_index, const emelb_window_layer** out,
                                           uint64_t* slot_capacity_bytes);
/* Host-side failure injection for tests: the next `count` slot loads report a
 * failed copy without touching the device. */
EMELB_API uint32_t emelb_window_fail_next_loads(emelb_window* w, int32_t count);
/* 1: bind does not try to page-lock the source (forces the staged route). */
EMELB_API uint32_t emelb_window_set_staged_only(emelb_window* w, int32_t staged_only);

#ifdef __cplusplus
}
#endif

#endif /* EMELB_WINDOW_H */
