// GGUF file image -> tensor table -> residency (include/emelb_gguf.h).
//
// One forward walk over the image serves both questions the reference asks of a
// file: "what storage does it need" (probe_requirements,
// src/emel/gguf/loader/detail.hpp:419-543) and "what does it hold"
// (parse_bound_storage, detail.hpp:545-733).  The walk hands each key/value pair
// and each tensor description to a sink; the probe's sink only keeps maxima, the
// opener's sink appends records.  The order of the checks, and with it which
// error a malformed image gets, is the reference's: a short or foreign header is
// parse_failed (under four bytes) or model_invalid; counts beyond 32 bits are
// capacity; a read past the end is parse_failed; an unknown value or tensor type,
// a bad general.alignment, more than four dimensions or a row that is not whole
// blocks is model_invalid; arithmetic that leaves 64 bits is capacity; a tensor
// whose offset is not the running padded offset is parse_failed; and the padded
// data must fit in the image.
//
// Host code only: the one device interaction is emelb_residency_upload.
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cstdint>
#include <cstring>
#include <new>
#include <vector>

#include "../../include/emelb_gguf.h"
#include "ctx.h"

namespace {

constexpr uint32_t kVersion = 3;            // detail.hpp:22
constexpr uint32_t kDefaultAlignment = 32;  // detail.hpp:23
constexpr uint32_t kMaxDims = 4;            // detail.hpp:24
constexpr uint32_t kValueTypes = 13;        // detail.hpp:39
constexpr uint64_t kU32Max = 0xffffffffull;
const char kAlignmentKey[] = "general.alignment";

// elements per block / bytes per block of each ggml tensor type the reference
// sizes (detail.hpp:48-84); {0, 0} = unknown
struct BlockLayout {
  uint16_t elems, bytes;
};
BlockLayout block_layout(uint32_t t) {
  static const BlockLayout table[40] = {
      {1, 4},     {1, 2},     {32, 18},  {32, 20},  {0, 0},    {0, 0},    {32, 22},   {32, 24},
      {32, 34},   {32, 36},   {256, 84}, {256, 110}, {256, 144}, {256, 176}, {256, 210}, {256, 292},
      {256, 66},  {256, 74},  {256, 98}, {256, 50}, {32, 18},  {256, 110}, {256, 82},  {256, 136},
      {1, 1},     {1, 2},     {1, 4},    {1, 8},    {1, 8},    {256, 56}, {1, 2},     {0, 0},
      {0, 0},     {0, 0},     {256, 54}, {256, 66}, {0, 0},    {0, 0},    {0, 0},     {32, 17}};
  return t < 40 ? table[t] : BlockLayout{0, 0};
}
// the two row-group-packed Q4_K layouts: 8 rows x 256 columns per 1152 bytes
// (detail.hpp:86-89, 135-163)
bool is_row_group_packed(uint32_t t) { return t == 41 || t == 42; }

uint32_t scalar_bytes(uint32_t value_type) {  // detail.hpp:91-106
  switch (value_type) {
    case EMELB_GGUF_T_UINT8: case EMELB_GGUF_T_INT8: case EMELB_GGUF_T_BOOL: return 1;
    case EMELB_GGUF_T_UINT16: case EMELB_GGUF_T_INT16: return 2;
    case EMELB_GGUF_T_UINT32: case EMELB_GGUF_T_INT32: case EMELB_GGUF_T_FLOAT32: return 4;
    case EMELB_GGUF_T_UINT64: case EMELB_GGUF_T_INT64: case EMELB_GGUF_T_FLOAT64: return 8;
    default: return 0;
  }
}

// *out is written only when the result fits (it may alias an operand)
bool checked_add(uint64_t a, uint64_t b, uint64_t* out) {
  uint64_t r;
  if (__builtin_add_overflow(a, b, &r)) return false;
  *out = r;
  return true;
}
bool checked_mul(uint64_t a, uint64_t b, uint64_t* out) {
  uint64_t r;
  if (__builtin_mul_overflow(a, b, &r)) return false;
  *out = r;
  return true;
}
bool round_up(uint64_t v, uint32_t alignment, uint64_t* out) {
  const uint64_t rem = v % alignment;
  if (rem == 0) { *out = v; return true; }
  return checked_add(v, alignment - rem, out);
}

// little-endian cursor that never reads past the image (detail.hpp:179-248)
struct Cursor {
  const uint8_t* base;
  uint64_t size;
  uint64_t at = 0;

  bool has(uint64_t n) const { return n <= size && at <= size - n; }
  bool u32(uint32_t* v) {
    if (!has(4)) return false;
    *v = uint32_t(base[at]) | uint32_t(base[at + 1]) << 8 | uint32_t(base[at + 2]) << 16 | uint32_t(base[at + 3]) << 24;
    at += 4;
    return true;
  }
  bool u64(uint64_t* v) {
    uint32_t lo, hi;
    if (!has(8)) return false;
    u32(&lo);
    u32(&hi);
    *v = uint64_t(hi) << 32 | lo;
    return true;
  }
  bool skip(uint64_t n) {
    if (!has(n)) return false;
    at += n;
    return true;
  }
  // u64 length + bytes
  bool str(const char** s, uint64_t* len) {
    if (!u64(len) || !has(*len)) return false;
    *s = reinterpret_cast<const char*>(base + at);
    at += *len;
    return true;
  }
};

// one key/value payload (detail.hpp:288-370); *alignment changes only for a valid
// general.alignment
uint32_t walk_value(Cursor& c, uint32_t type, const char* key, uint64_t key_len, uint32_t* alignment) {
  if (type >= kValueTypes) return EMELB_GGUF_MODEL_INVALID;
  const char* s;
  uint64_t n;
  if (type == EMELB_GGUF_T_STRING) return c.str(&s, &n) ? EMELB_GGUF_OK : EMELB_GGUF_PARSE_FAILED;
  if (type == EMELB_GGUF_T_ARRAY) {
    uint32_t elem_type;
    uint64_t count, payload;
    if (!c.u32(&elem_type) || !c.u64(&count)) return EMELB_GGUF_PARSE_FAILED;
    if (elem_type >= kValueTypes || elem_type == EMELB_GGUF_T_ARRAY) return EMELB_GGUF_MODEL_INVALID;
    if (elem_type == EMELB_GGUF_T_STRING) {
      for (uint64_t i = 0; i < count; ++i)
        if (!c.str(&s, &n)) return EMELB_GGUF_PARSE_FAILED;
      return EMELB_GGUF_OK;
    }
    if (!checked_mul(count, scalar_bytes(elem_type), &payload)) return EMELB_GGUF_CAPACITY;
    return c.skip(payload) ? EMELB_GGUF_OK : EMELB_GGUF_PARSE_FAILED;
  }
  const uint32_t width = scalar_bytes(type);
  if (key_len == sizeof(kAlignmentKey) - 1 && std::memcmp(key, kAlignmentKey, key_len) == 0) {
    uint32_t a;
    if (type != EMELB_GGUF_T_UINT32) return EMELB_GGUF_MODEL_INVALID;
    if (!c.u32(&a)) return EMELB_GGUF_PARSE_FAILED;
    if (a == 0 || (a & (a - 1)) != 0) return EMELB_GGUF_MODEL_INVALID;
    *alignment = a;
    return EMELB_GGUF_OK;
  }
  return c.skip(width) ? EMELB_GGUF_OK : EMELB_GGUF_PARSE_FAILED;
}

// bytes of a tensor's data (detail.hpp:135-163, 372-403)
uint32_t tensor_bytes(const uint64_t dims[4], uint32_t n_dims, uint32_t type, uint64_t* out) {
  if (is_row_group_packed(type)) {
    if (n_dims < 2 || n_dims > kMaxDims || dims[0] % 256 != 0) return EMELB_GGUF_MODEL_INVALID;
    uint64_t rows = 1, cells;
    for (uint32_t d = 1; d < n_dims; ++d)
      if (!checked_mul(rows, dims[d], &rows)) return EMELB_GGUF_CAPACITY;
    const uint64_t groups = rows / 8 + (rows % 8 != 0);
    if (!checked_mul(groups, dims[0] / 256, &cells) || !checked_mul(cells, 1152, out)) return EMELB_GGUF_CAPACITY;
    return EMELB_GGUF_OK;
  }
  const BlockLayout l = block_layout(type);
  if (l.elems == 0) return EMELB_GGUF_MODEL_INVALID;
  if ((n_dims == 0 ? 1 : dims[0]) % l.elems != 0) return EMELB_GGUF_MODEL_INVALID;
  uint64_t elems = 1;
  for (uint32_t d = 0; d < n_dims; ++d)
    if (!checked_mul(elems, dims[d], &elems)) return EMELB_GGUF_CAPACITY;
  return checked_mul(elems / l.elems, l.bytes, out) ? EMELB_GGUF_OK : EMELB_GGUF_CAPACITY;
}

struct Walked {
  emelb_gguf_requirements req{};
  uint32_t alignment = kDefaultAlignment;
  uint64_t data_section = 0;
};

// Sink: void kv(const emelb_gguf_kv&); void tensor(const emelb_gguf_tensor&)  (data/file_offset unset)
template <class Sink>
uint32_t walk(const uint8_t* image, uint64_t bytes, Sink& sink, Walked* w) {
  Cursor c{image, bytes};
  uint32_t version = 0;
  uint64_t n_tensors = 0, n_kv = 0;
  const bool header = c.has(4) && std::memcmp(image, "GGUF", 4) == 0 && c.skip(4) && c.u32(&version) &&
                      c.u64(&n_tensors) && c.u64(&n_kv) && version == kVersion;
  if (!header) return bytes < 4 ? EMELB_GGUF_PARSE_FAILED : EMELB_GGUF_MODEL_INVALID;
  if (n_tensors > kU32Max || n_kv > kU32Max) return EMELB_GGUF_CAPACITY;
  w->req.tensor_count = uint32_t(n_tensors);
  w->req.kv_count = uint32_t(n_kv);

  uint32_t alignment = kDefaultAlignment;
  for (uint64_t i = 0; i < n_kv; ++i) {
    const char* key;
    uint64_t key_len;
    uint32_t type;
    if (!c.str(&key, &key_len) || !c.u32(&type)) return EMELB_GGUF_PARSE_FAILED;
    if (key_len > kU32Max) return EMELB_GGUF_CAPACITY;
    const uint64_t value_at = c.at;
    if (const uint32_t err = walk_value(c, type, key, key_len, &alignment)) return err;
    const uint64_t value_len = c.at - value_at;
    if (value_len > kU32Max) return EMELB_GGUF_CAPACITY;
    if (w->req.max_key_bytes < key_len) w->req.max_key_bytes = uint32_t(key_len);
    if (w->req.max_value_bytes < value_len) w->req.max_value_bytes = uint32_t(value_len);
    sink.kv(emelb_gguf_kv{key, uint32_t(key_len), type, image + value_at, uint32_t(value_len)});
  }

  uint64_t running = 0;  // offset the next tensor must carry
  for (uint64_t i = 0; i < n_tensors; ++i) {
    const char* name;
    uint64_t name_len, dims[4] = {1, 1, 1, 1}, offset, size = 0, padded;
    uint32_t n_dims, type;
    if (!c.str(&name, &name_len) || !c.u32(&n_dims)) return EMELB_GGUF_PARSE_FAILED;
    if (name_len > kU32Max) return EMELB_GGUF_CAPACITY;
    if (n_dims > kMaxDims) return EMELB_GGUF_MODEL_INVALID;
    for (uint32_t d = 0; d < n_dims; ++d)
      if (!c.u64(&dims[d])) return EMELB_GGUF_PARSE_FAILED;
    if (!c.u32(&type) || !c.u64(&offset)) return EMELB_GGUF_PARSE_FAILED;
    if (const uint32_t err = tensor_bytes(dims, n_dims, type, &size)) return err;
    if (!checked_add(w->req.tensor_data_bytes, size, &w->req.tensor_data_bytes)) return EMELB_GGUF_CAPACITY;
    if (offset != running) return EMELB_GGUF_PARSE_FAILED;
    if (!round_up(size, alignment, &padded) || !checked_add(running, padded, &running)) return EMELB_GGUF_CAPACITY;
    emelb_gguf_tensor t{};
    t.name = name;
    t.name_length = uint32_t(name_len);
    t.type = int32_t(type);
    t.n_dims = int32_t(n_dims);
    for (int d = 0; d < 4; ++d) t.dims[d] = int64_t(dims[d]);
    t.data_offset = offset;
    t.data_size = size;
    sink.tensor(t);
  }

  uint64_t data_section, need;
  if (!round_up(c.at, alignment, &data_section) || data_section > bytes) return EMELB_GGUF_PARSE_FAILED;
  if (!checked_add(data_section, running, &need)) return EMELB_GGUF_CAPACITY;
  if (need > bytes) return EMELB_GGUF_PARSE_FAILED;
  w->alignment = alignment;
  w->data_section = data_section;
  return EMELB_GGUF_OK;
}

struct CountingSink {
  void kv(const emelb_gguf_kv&) {}
  void tensor(const emelb_gguf_tensor&) {}
};

}  // namespace

struct emelb_gguf {
  const uint8_t* image = nullptr;
  uint64_t bytes = 0;
  void* mapping = nullptr;  // non-null when the handle owns an mmap of `bytes`
  int fd = -1;              // the mapped file, kept open so that uploads can read it without page faults
  Walked walked;
  std::vector<emelb_gguf_kv> kvs;
  std::vector<emelb_gguf_tensor> tensors;

  void kv(const emelb_gguf_kv& e) { kvs.push_back(e); }
  void tensor(const emelb_gguf_tensor& t) { tensors.push_back(t); }
};

namespace {

bool same_text(const char* a, uint32_t a_len, const char* b) {
  return std::strlen(b) == a_len && std::memcmp(a, b, a_len) == 0;
}

}  // namespace

extern "C" {

uint32_t emelb_gguf_probe(const uint8_t* image, uint64_t bytes, emelb_gguf_requirements* out) {
  // guard::probe_valid_request: an image and somewhere to put the answer
  if (!image || bytes == 0 || !out) return EMELB_GGUF_INVALID_REQUEST;
  CountingSink sink;
  Walked w;
  const uint32_t err = walk(image, bytes, sink, &w);
  // on failure the counts read so far stay visible, as in the reference
  *out = w.req;
  return err;
}

uint32_t emelb_gguf_open_image(const uint8_t* image, uint64_t bytes, emelb_gguf** out) {
  if (!image || bytes == 0 || !out) return EMELB_GGUF_INVALID_REQUEST;
  *out = nullptr;
  emelb_gguf* g = new (std::nothrow) emelb_gguf;
  if (!g) return EMELB_GGUF_CAPACITY;
  g->image = image;
  g->bytes = bytes;
  uint32_t err;
  try {
    err = walk(image, bytes, *g, &g->walked);
  } catch (const std::bad_alloc&) {
    err = EMELB_GGUF_CAPACITY;
  }
  if (err != EMELB_GGUF_OK) {
    delete g;
    return err;
  }
  // detail.hpp:714-730: absolute offsets, each span inside the image
  for (emelb_gguf_tensor& t : g->tensors) {
    uint64_t end;
    if (!checked_add(g->walked.data_section, t.data_offset, &t.file_offset) ||
        !checked_add(t.file_offset, t.data_size, &end)) {
      delete g;
      return EMELB_GGUF_CAPACITY;
    }
    if (end > bytes) {
      delete g;
      return EMELB_GGUF_PARSE_FAILED;
    }
    t.data = image + t.file_offset;
  }
  *out = g;
  return EMELB_GGUF_OK;
}

uint32_t emelb_gguf_open_file(const char* path, emelb_gguf** out) {
  if (!path || !out) return EMELB_GGUF_INVALID_REQUEST;
  *out = nullptr;
  const int fd = ::open(path, O_RDONLY | O_CLOEXEC);
  if (fd < 0) return EMELB_GGUF_INVALID_REQUEST;
  struct stat st;
  if (::fstat(fd, &st) != 0 || !S_ISREG(st.st_mode)) {
    ::close(fd);
    return EMELB_GGUF_INVALID_REQUEST;
  }
  if (st.st_size == 0) {
    ::close(fd);
    return EMELB_GGUF_INVALID_REQUEST;  // an empty image is no request (guard::has_file_image)
  }
  const uint64_t bytes = uint64_t(st.st_size);
  void* m = ::mmap(nullptr, bytes, PROT_READ, MAP_PRIVATE, fd, 0);
  if (m == MAP_FAILED) {
    ::close(fd);
    return EMELB_GGUF_INTERNAL_ERROR;
  }
  const uint32_t err = emelb_gguf_open_image(static_cast<const uint8_t*>(m), bytes, out);
  if (err != EMELB_GGUF_OK) {
    ::munmap(m, bytes);
    ::close(fd);
    return err;
  }
  (*out)->mapping = m;
  (*out)->fd = fd;
  return EMELB_GGUF_OK;
}

uint32_t emelb_gguf_close(emelb_gguf* g) {
  if (!g) return EMELB_GGUF_INVALID_REQUEST;
  if (g->mapping) ::munmap(g->mapping, g->bytes);
  if (g->fd >= 0) ::close(g->fd);
  delete g;
  return EMELB_GGUF_OK;
}

uint32_t emelb_gguf_get_requirements(const emelb_gguf* g, emelb_gguf_requirements* out) {
  if (!g || !out) return EMELB_GGUF_INVALID_REQUEST;
  *out = g->walked.req;
  return EMELB_GGUF_OK;
}

uint32_t emelb_gguf_layout(const emelb_gguf* g, uint32_t* alignment_out, uint64_t* data_section_offset_out) {
  if (!g) return EMELB_GGUF_INVALID_REQUEST;
  if (alignment_out) *alignment_out = g->walked.alignment;
  if (data_section_offset_out) *data_section_offset_out = g->walked.data_section;
  return EMELB_GGUF_OK;
}

uint32_t emelb_gguf_tensor_at(const emelb_gguf* g, uint32_t index, emelb_gguf_tensor* out) {
  if (!g || !out || index >= g->tensors.size()) return EMELB_GGUF_INVALID_REQUEST;
  *out = g->tensors[index];
  return EMELB_GGUF_OK;
}

uint32_t emelb_gguf_kv_at(const emelb_gguf* g, uint32_t index, emelb_gguf_kv* out) {
  if (!g || !out || index >= g->kvs.size()) return EMELB_GGUF_INVALID_REQUEST;
  *out = g->kvs[index];
  return EMELB_GGUF_OK;
}

int32_t emelb_gguf_find_tensor(const emelb_gguf* g, const char* name) {
  if (!g || !name) return -1;
  for (size_t i = 0; i < g->tensors.size(); ++i)
    if (same_text(g->tensors[i].name, g->tensors[i].name_length, name)) return int32_t(i);
  return -1;
}

int32_t emelb_gguf_find_kv(const emelb_gguf* g, const char* key) {
  if (!g || !key) return -1;
  for (size_t i = 0; i < g->kvs.size(); ++i)
    if (same_text(g->kvs[i].key, g->kvs[i].key_length, key)) return int32_t(i);
  return -1;
}

uint32_t emelb_gguf_upload(emelb_ctx* ctx, const emelb_gguf* g, uint32_t tensor_index, int32_t tensor_id,
                           const void** dev_out) {
  if (!ctx || !g || tensor_index >= g->tensors.size()) return EMELB_GGUF_INVALID_REQUEST;
  const emelb_gguf_tensor& t = g->tensors[tensor_index];
  if (t.data_size == 0) return EMELB_GGUF_INVALID_REQUEST;
  emelb::UploadSpan span{tensor_id, t.data, t.data_size, t.type, t.file_offset, nullptr};
  const uint32_t err = emelb::residency_upload_many(ctx, &span, 1, g->fd);
  if (err == EMELB_OK && dev_out) *dev_out = span.dev;
  if (err == EMELB_OK) return EMELB_GGUF_OK;
  // a tensor id that is already resident is the caller's mistake; anything else is the device's
  return err == EMELB_INVALID_REQUEST ? EMELB_GGUF_INVALID_REQUEST : EMELB_GGUF_INTERNAL_ERROR;
}

uint32_t emelb_gguf_upload_all(emelb_ctx* ctx, const emelb_gguf* g, int32_t first_tensor_id) {
  if (!ctx || !g) return EMELB_GGUF_INVALID_REQUEST;
  std::vector<emelb::UploadSpan> spans;
  try {
    spans.reserve(g->tensors.size());
    for (size_t i = 0; i < g->tensors.size(); ++i) {
      const emelb_gguf_tensor& t = g->tensors[i];
      if (t.data_size == 0) continue;  // nothing to hold in HBM
      spans.push_back(emelb::UploadSpan{int32_t(first_tensor_id + int32_t(i)), t.data, t.data_size, t.type, t.file_offset, nullptr});
    }
  } catch (const std::bad_alloc&) {
    return EMELB_GGUF_CAPACITY;
  }
  if (spans.empty()) return EMELB_GGUF_OK;
  const uint32_t err = emelb::residency_upload_many(ctx, spans.data(), spans.size(), g->fd);
  if (err == EMELB_OK) return EMELB_GGUF_OK;
  return err == EMELB_INVALID_REQUEST ? EMELB_GGUF_INVALID_REQUEST : EMELB_GGUF_INTERNAL_ERROR;
}

uint32_t emelb_gguf_upload_rows(emelb_ctx* ctx, const emelb_gguf* g, uint32_t tensor_index, int32_t tensor_id,
                                uint64_t first_row, uint64_t rows, const void** host_out, const void** dev_out) {
  if (!ctx || !g || tensor_index >= g->tensors.size() || rows == 0) return EMELB_GGUF_INVALID_REQUEST;
  const emelb_gguf_tensor& t = g->tensors[tensor_index];
  const BlockLayout l = block_layout(uint32_t(t.type));
  if (l.elems == 0 || t.n_dims < 2) return EMELB_GGUF_INVALID_REQUEST;
  const uint64_t row_bytes = uint64_t(t.dims[0]) / l.elems * l.bytes;  // whole blocks: checked when the file was opened
  if (row_bytes == 0) return EMELB_GGUF_INVALID_REQUEST;
  const uint64_t total_rows = t.data_size / row_bytes;
  if (first_row > total_rows || rows > total_rows - first_row) return EMELB_GGUF_INVALID_REQUEST;
  const uint8_t* host = static_cast<const uint8_t*>(t.data) + first_row * row_bytes;
  emelb::UploadSpan span{tensor_id, host, rows * row_bytes, t.type, t.file_offset + first_row * row_bytes, nullptr};
  const uint32_t err = emelb::residency_upload_many(ctx, &span, 1, g->fd);
  if (err == EMELB_OK && dev_out) *dev_out = span.dev;
  if (err != EMELB_OK) return err == EMELB_INVALID_REQUEST ? EMELB_GGUF_INVALID_REQUEST : EMELB_GGUF_INTERNAL_ERROR;
  if (host_out) *host_out = host;
  return EMELB_GGUF_OK;
}

}  // extern "C"
