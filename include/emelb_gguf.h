/*
 * emelb_gguf.h — GGUF file image -> tensor table -> HBM residency.
 *
 * The reference reads a model in three steps: gguf::loader probes a file image
 * for its storage requirements, the caller binds storage, and the loader parses
 * the key/value section and the tensor table into tensor_record entries whose
 * `data` points into the (mmap'd) image (src/emel/gguf/loader/events.hpp:49-96,
 * src/emel/gguf/loader/detail.hpp:419-733, src/emel/model/data.hpp:123-134);
 * io::mmap maps tensor spans of the file (src/emel/io/mmap/events.hpp:23-44).
 * Here the same validation and the same records come out of one call, with the
 * storage owned by the library, and emelb_gguf_upload hands a tensor's span of
 * the mapping to the residency table of a backend context: the bytes go from
 * the page cache to HBM unchanged, and the mapping address stays the key a
 * later emelb_view may carry.
 *
 * Every call returns the loader's error bitmask
 * (src/emel/gguf/loader/errors.hpp:7-15), not the kernel one.
 */
#ifndef EMELB_GGUF_H
#define EMELB_GGUF_H

#include "emelb.h"

#ifdef __cplusplus
extern "C" {
#endif

/* src/emel/gguf/loader/errors.hpp:7-15 */
enum {
  EMELB_GGUF_OK = 0u,
  EMELB_GGUF_INVALID_REQUEST = 1u << 0,
  EMELB_GGUF_MODEL_INVALID = 1u << 1,
  EMELB_GGUF_CAPACITY = 1u << 2,
  EMELB_GGUF_PARSE_FAILED = 1u << 3,
  EMELB_GGUF_INTERNAL_ERROR = 1u << 4,
  EMELB_GGUF_UNTRACKED = 1u << 5
};

/* GGUF metadata value types (src/emel/gguf/loader/detail.hpp:26-39) */
enum {
  EMELB_GGUF_T_UINT8 = 0, EMELB_GGUF_T_INT8 = 1, EMELB_GGUF_T_UINT16 = 2, EMELB_GGUF_T_INT16 = 3,
  EMELB_GGUF_T_UINT32 = 4, EMELB_GGUF_T_INT32 = 5, EMELB_GGUF_T_FLOAT32 = 6, EMELB_GGUF_T_BOOL = 7,
  EMELB_GGUF_T_STRING = 8, EMELB_GGUF_T_ARRAY = 9, EMELB_GGUF_T_UINT64 = 10, EMELB_GGUF_T_INT64 = 11,
  EMELB_GGUF_T_FLOAT64 = 12
};

/* requirements: src/emel/gguf/loader/events.hpp:13-19 */
typedef struct emelb_gguf_requirements {
  uint32_t tensor_count;
  uint32_t kv_count;
  uint32_t max_key_bytes;
  uint32_t max_value_bytes;
  uint64_t tensor_data_bytes;
} emelb_gguf_requirements;

/* tensor_record: src/emel/model/data.hpp:123-134.  `name` is not terminated;
 * data_offset is relative to the data section, file_offset to the image. */
typedef struct emelb_gguf_tensor {
  const char* name;
  uint32_t name_length;
  int32_t type;
  int32_t n_dims;
  int64_t dims[4];
  uint64_t data_offset;
  uint64_t file_offset;
  uint64_t data_size;
  const void* data;
} emelb_gguf_tensor;

/* kv_entry: src/emel/gguf/loader/events.hpp:21-27.  `value` is the serialized
 * payload as it stands in the file (little-endian scalar; u64 length + bytes for
 * a string; u32 element type, u64 count, elements for an array). */
typedef struct emelb_gguf_kv {
  const char* key;
  uint32_t key_length;
  uint32_t value_type;
  const uint8_t* value;
  uint32_t value_length;
} emelb_gguf_kv;

typedef struct emelb_gguf emelb_gguf;

/* replaces event::probe -> probe_requirements (detail.hpp:419-543): validates the
 * whole header, key/value section and tensor table; nothing is allocated */
EMELB_API uint32_t emelb_gguf_probe(const uint8_t* image, uint64_t bytes,
                                    emelb_gguf_requirements* out);

/* replaces event::bind_storage + event::parse (detail.hpp:545-733) with storage
 * owned by the handle.  The image must outlive the handle. */
EMELB_API uint32_t emelb_gguf_open_image(const uint8_t* image, uint64_t bytes,
                                         emelb_gguf** out);
/* maps the file read-only (the whole file, one mapping) and opens the mapping */
EMELB_API uint32_t emelb_gguf_open_file(const char* path, emelb_gguf** out);
EMELB_API uint32_t emelb_gguf_close(emelb_gguf* g);

EMELB_API uint32_t emelb_gguf_get_requirements(const emelb_gguf* g,
                                               emelb_gguf_requirements* out);
/* general.alignment in force for the tensor data (32 when the key is absent)
 * and the offset of the data section in the image */
EMELB_API uint32_t emelb_gguf_layout(const emelb_gguf* g, uint32_t* alignment_out,
                                     uint64_t* data_section_offset_out);
EMELB_API uint32_t emelb_gguf_tensor_at(const emelb_gguf* g, uint32_t index,
                                        emelb_gguf_tensor* out);
EMELB_API uint32_t emelb_gguf_kv_at(const emelb_gguf* g, uint32_t index,
                                    emelb_gguf_kv* out);
/* first entry with exactly this name / key; -1 when absent */
EMELB_API int32_t emelb_gguf_find_tensor(const emelb_gguf* g, const char* name);
EMELB_API int32_t emelb_gguf_find_kv(const emelb_gguf* g, const char* key);

/* the tensor's bytes -> HBM through the context's residency table
 * (emelb_residency_upload with host = the tensor's address in the image):
 * replaces routing the record through model::tensor with the external_buffer
 * strategy (src/emel/io/loader/events.hpp:25-31).  dev_out may be null. */
EMELB_API uint32_t emelb_gguf_upload(emelb_ctx* ctx, const emelb_gguf* g,
                                     uint32_t tensor_index, int32_t tensor_id,
                                     const void** dev_out);

/* every tensor of the file in one pipelined pass (tensor i gets id
 * first_tensor_id + i; tensors without data are skipped).  All or nothing: on an
 * error no tensor of the file has become resident through this call. */
EMELB_API uint32_t emelb_gguf_upload_all(emelb_ctx* ctx, const emelb_gguf* g,
                                         int32_t first_tensor_id);

/* rows [first_row, first_row + rows) of a tensor of two or more dimensions (a row
 * is dims[0] elements; rows count over the remaining dimensions): what one rank
 * of a row-sharded product holds (src/emel/kernel/matmul/actions.hpp:49-66).
 * host_out receives the interval's address in the image, the key to bind it by.
 * The row-group-packed types (41, 42) do not slice by rows: invalid_request. */
EMELB_API uint32_t emelb_gguf_upload_rows(emelb_ctx* ctx, const emelb_gguf* g,
                                          uint32_t tensor_index, int32_t tensor_id,
                                          uint64_t first_row, uint64_t rows,
                                          const void** host_out, const void** dev_out);

#ifdef __cplusplus
}
#endif
#endif /* EMELB_GGUF_H */
