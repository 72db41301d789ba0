// C-ABI of the backend (include/emelb.h): context, residency table, request
// guards and op dispatch.  No entry point allocates after emelb_create /
// emelb_residency_upload / emelb_device_alloc.
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <map>
#include <new>

#include "../../include/emelb.h"
#include "ctx.h"

using namespace emelb;

namespace {

// ------------------------------------------------------------------ guards
// Restates validate_dispatch_request + can_run_* of the reference for the
// dtypes on this path (src/emel/kernel/detail.hpp:1545-1598, 1709-1749,
// 1792-1927, 3573-3606, 3843-3872, 4346-4390).
bool is_32_type(int t) { return t == T_Q4_0 || t == T_Q8_0; }
bool is_native_quant(int t) { return is_k_type(t) || is_32_type(t); }
// integer bytes per element; 0 for the sub-byte formats, as in the reference
uint64_t elem_size(int t) {
  switch (t) {
    case T_F32: return 4;
    case T_F16: return 2;
    case T_I32: return 4;
    case T_Q8_0: return Q8_0_BYTES / 32;
    case T_Q8_K: return Q8_K_BYTES / 256;
    default: return 0;
  }
}
bool is_supported(int t) { return t == T_F32 || t == T_F16 || is_native_quant(t) || t == T_Q8_K; }
uint64_t row_bytes_of(int t, uint64_t cols) {
  const uint64_t be = block_elems(t);
  if (be == 0 || cols % be != 0) return 0;
  return cols / be * block_bytes(t);
}
bool valid_layout(const emelb_view& v) {
  const uint64_t es = elem_size(v.type);
  const bool explicit_stride = v.nb[0] != 0;
  const bool aligned = es != 0 && explicit_stride && v.nb[0] >= es && v.nb[0] % es == 0;
  bool dims_ok = true;
  for (int i = 0; i < 4; ++i) dims_ok = dims_ok && !(v.ne[i] > 1 && v.nb[i] == 0);
  return es != 0 && (!explicit_stride || (aligned && dims_ok));
}
uint64_t stride_bytes(const emelb_view& v, int dim) {
  uint64_t s = elem_size(v.type);
  for (int i = 0; i < dim; ++i) s *= v.ne[i];
  return v.nb[0] != 0 ? v.nb[dim] : s;
}
bool dense(const emelb_view& v) {
  uint64_t expect = elem_size(v.type);
  bool ok = true;
  for (int i = 0; i < 4; ++i) {
    ok = ok && stride_bytes(v, i) == expect;
    expect *= v.ne[i];
  }
  return valid_layout(v) && ok;
}
uint64_t elem_count(const emelb_view& v) { return v.ne[0] * v.ne[1] * v.ne[2] * v.ne[3]; }
bool required_plain(const emelb_view& v) {
  return v.data != nullptr && is_supported(v.type) && valid_layout(v) && elem_count(v) > 0;
}
bool required_src0_matmul(const emelb_view& s) {
  if (is_native_quant(s.type)) {
    const uint64_t rb = row_bytes_of(s.type, s.ne[0]);
    return s.data && rb != 0 && s.ne[1] != 0 && s.ne[2] == 1 && s.ne[3] == 1 && s.nb[0] == 1 && s.nb[1] == rb &&
           s.nb[2] == rb * s.ne[1] && s.nb[3] == s.nb[2];
  }
  return required_plain(s);
}

// the pre-quantized vector form of src1 (one activation vector already in
// Q8_K / Q8_0 blocks): ne = {1, K}, nb = {1, row_bytes, row_bytes, row_bytes}
// (src/emel/kernel/aarch64/actions.hpp:1471-1503, 964-997)
bool prequantized_src1(const emelb_op& r) {
  const int wt = r.src0.type, at = r.src1.type;
  if (!((is_k_type(wt) && at == T_Q8_K) || (is_32_type(wt) && at == T_Q8_0))) return false;
  const uint64_t k = r.src0.ne[0];
  const uint64_t rb = row_bytes_of(at, k);
  return r.src1.data && rb != 0 && r.src1.ne[0] == 1 && r.src1.ne[1] == k && r.src1.ne[2] == 1 && r.src1.ne[3] == 1 &&
         r.src1.nb[0] == 1 && r.src1.nb[1] == rb && r.src1.nb[2] == rb && r.src1.nb[3] == rb;
}

bool quant_matmul_common(const emelb_op& r, uint64_t n_expected_dst0, uint64_t m_expected_dst1, bool allow_preq) {
  const uint64_t k = r.src0.ne[0], m = r.src0.ne[1];
  const int t = r.src0.type;
  const uint64_t be = block_elems(t);
  const uint64_t lim = is_32_type(t) ? MAX_Q8_0_BLOCKS : (is_k_type(t) ? MAX_Q8_K_BLOCKS : 0);
  const bool shape = r.src1.ne[1] == k && r.dst.ne[0] == n_expected_dst0 && r.dst.ne[1] == m_expected_dst1 &&
                     r.src0.ne[2] == 1 && r.src0.ne[3] == 1 && r.src1.ne[2] == 1 && r.src1.ne[3] == 1 &&
                     r.dst.ne[2] == 1 && r.dst.ne[3] == 1;
  const bool src1_ok = (r.src1.type == T_F32 && dense(r.src1)) || (allow_preq && prequantized_src1(r));
  const bool q = is_native_quant(t) && src1_ok && r.dst.type == T_F32 && be != 0 && k % be == 0 && k / be <= lim &&
                 dense(r.dst) && r.src0.nb[0] == 1 && r.src0.nb[1] == row_bytes_of(t, k) &&
                 r.src0.nb[2] == r.src0.nb[1] * m && r.src0.nb[3] == r.src0.nb[2];
  return shape && q;
}

bool can_run_mul_mat(const emelb_op& r) {
  const bool preq = prequantized_src1(r);
  if (!(required_src0_matmul(r.src0) && (preq || required_plain(r.src1)) && required_plain(r.dst))) return false;
  if (r.op_params_size > 64) return false;
  const uint64_t k = r.src0.ne[0], m = r.src0.ne[1], n = r.src1.ne[0];
  if (k == 0 || m == 0 || n == 0) return false;
  return quant_matmul_common(r, n, m, true);
}

bool can_run_mul_mat_argmax(const emelb_op& r) {
  if (!(required_src0_matmul(r.src0) && required_plain(r.src1) && required_plain(r.dst))) return false;
  if (r.op_params_size > 64) return false;
  const uint64_t k = r.src0.ne[0], m = r.src0.ne[1], n = r.src1.ne[0];
  if (k == 0 || m == 0 || n != 1 || r.index_out == nullptr) return false;
  return quant_matmul_common(r, 1, 1, false);
}

float fa_scale(const emelb_op& r) {
  if (r.op_params_size >= 4) { float s; std::memcpy(&s, r.op_params, 4); return s; }
  const float hd = (float)r.src0.ne[0];
  return hd > 0.0f ? 1.0f / std::sqrt(hd) : 1.0f;
}
uint64_t fa_masked_total(const emelb_op& r) {
  if (r.op_params_size >= 8) { uint32_t t; std::memcpy(&t, r.op_params + 4, 4); return t; }
  return r.src1.ne[1];
}

bool can_run_flash(const emelb_op& r) {
  if (!(required_plain(r.src0) && required_plain(r.src1) && required_plain(r.dst))) return false;
  if (r.op_params_size > 64) return false;
  const uint64_t hd = r.src0.ne[0], qc = r.src0.ne[1], hc = r.src0.ne[2], T = r.src1.ne[1], kvh = r.src1.ne[2];
  const bool types = r.src0.type == T_F32 && r.src1.type == T_F16 && r.src2.type == T_F16 && r.dst.type == T_F32;
  const bool dims = hd != 0 && qc == 1 && hc != 0 && T != 0 && kvh != 0;
  const bool shape = r.src1.ne[0] == hd && r.src2.ne[0] == hd && r.src2.ne[1] == T && r.src2.ne[2] == kvh &&
                     r.dst.ne[0] == hd && r.dst.ne[1] == qc && r.dst.ne[2] == hc && r.src0.ne[3] == 1 &&
                     r.src1.ne[3] == 1 && r.src2.ne[3] == 1 && r.dst.ne[3] == 1 && kvh != 0 && hc % (kvh ? kvh : 1) == 0;
  const bool layout = dense(r.src0) && valid_layout(r.src1) && valid_layout(r.src2) && dense(r.dst);
  const float scale = fa_scale(r);
  // head_dim <= 4096: the reference's workspace bound (src/emel/kernel/detail.hpp:170, 5219-5227)
  return types && dims && required_plain(r.src2) && shape && layout && fa_masked_total(r) >= T && std::isfinite(scale) &&
         scale > 0.0f && hd <= 4096;
}

// ------------------------------------------------------------------ pointers
// ---- op_rms_norm / op_rope / op_glu guards (src/emel/kernel/detail.hpp:4547-4565, 4650-4702, 5315-5335)
bool read_param_f32(const emelb_op& r, uint32_t slot, float* out) {
  if (((uint64_t)slot + 1) * 4 > r.op_params_size || r.op_params_size > 64) return false;
  std::memcpy(out, r.op_params + 4 * slot, 4);
  return true;
}
bool read_param_i32(const emelb_op& r, uint32_t slot, int32_t* out) {
  if (((uint64_t)slot + 1) * 4 > r.op_params_size || r.op_params_size > 64) return false;
  std::memcpy(out, r.op_params + 4 * slot, 4);
  return true;
}
bool same_shape(const emelb_view& a, const emelb_view& b) {
  return a.ne[0] == b.ne[0] && a.ne[1] == b.ne[1] && a.ne[2] == b.ne[2] && a.ne[3] == b.ne[3];
}
// has_required_src0 / has_required_dst of a plain op: data, a supported dtype, a valid layout, elements
bool required_tensor(const emelb_view& v) {
  const bool supported = is_supported(v.type) || v.type == T_I32;
  return v.data != nullptr && supported && valid_layout(v) && elem_count(v) > 0;
}
bool can_run_rms_norm(const emelb_op& r) {
  float eps = 0.0f;
  return required_tensor(r.src0) && required_tensor(r.dst) && r.op_params_size <= 64 && r.src0.ne[0] > 0 && same_shape(r.src0, r.dst) &&
         r.src0.type == T_F32 && r.dst.type == T_F32 && read_param_f32(r, 0, &eps) && std::isfinite(eps) && eps >= 0.0f;
}
struct RopeParams {
  int32_t n_dims = 0, mode = 0;
  float freq_base = 0.0f, freq_scale = 0.0f, ext_factor = 0.0f, attn_factor = 0.0f;
};
bool read_rope_params(const emelb_op& r, RopeParams* p) {
  return read_param_i32(r, 1, &p->n_dims) && read_param_i32(r, 2, &p->mode) && read_param_f32(r, 5, &p->freq_base) &&
         read_param_f32(r, 6, &p->freq_scale) && read_param_f32(r, 7, &p->ext_factor) && read_param_f32(r, 8, &p->attn_factor);
}
constexpr int32_t kRopeNorm = 0, kRopeNeox = 2;
bool can_run_rope(const emelb_op& r) {
  RopeParams p;
  // the positions are checked by the operator's own guard only (data, dtype, layout), not as a required source
  return required_tensor(r.src0) && r.src1.data != nullptr && valid_layout(r.src1) && required_tensor(r.dst) && r.op_params_size <= 64 &&
         read_rope_params(r, &p) && same_shape(r.src0, r.dst) && r.src0.ne[0] > 0 && r.src0.type == T_F32 && r.dst.type == T_F32 &&
         r.src1.type == T_I32 && r.src2.data == nullptr && r.src1.ne[0] == r.src0.ne[2] && p.n_dims > 0 && (p.n_dims % 2) == 0 &&
         (uint64_t)p.n_dims <= r.src0.ne[0] && p.ext_factor == 0.0f && std::isfinite(p.freq_base) && p.freq_base > 0.0f &&
         std::isfinite(p.freq_scale) && p.freq_scale > 0.0f && std::isfinite(p.attn_factor);
}

enum class Where { device, host, unknown };

// device ranges this context allocated itself are known without a driver query
bool known_device(const emelb_ctx* c, const void* p) {
  const uintptr_t a = reinterpret_cast<uintptr_t>(p);
  auto it = c->dev_ranges.upper_bound(a);
  if (it == c->dev_ranges.begin()) return false;
  --it;
  return a < it->first + it->second;
}

Where classify(const emelb_ctx* c, const void* p) {
  if (known_device(c, p)) return Where::device;
  cudaPointerAttributes at{};
  if (cudaPointerGetAttributes(&at, p) != cudaSuccess) {
    cudaGetLastError();
    return Where::unknown;
  }
  if (at.type == cudaMemoryTypeDevice || at.type == cudaMemoryTypeManaged) return Where::device;
  return Where::host;  // registered (pinned) or plain pageable host memory
}

// host span registered through emelb_residency_upload -> its device copy
const void* resident_lookup(const emelb_ctx* c, const void* host) {
  const uintptr_t a = reinterpret_cast<uintptr_t>(host);
  auto it = c->by_host.upper_bound(a);
  if (it == c->by_host.begin()) return nullptr;
  --it;
  const Resident& r = c->residents.at(it->second);
  if (r.state != EMELB_LIFECYCLE_RESIDENT || a >= it->first + r.bytes) return nullptr;
  return static_cast<const uint8_t*>(r.dev) + (a - it->first);
}

bool cuda_ok(emelb_ctx* c, cudaError_t e) {
  if (e == cudaSuccess) return true;
  c->last_cuda_error = (int)e;
  cudaGetLastError();
  return false;
}

// weights: device pointer, or a host pointer inside a resident span
const void* resolve_weights(emelb_ctx* c, const void* p) {
  if (const void* d = resident_lookup(c, p)) return d;
  return classify(c, p) == Where::device ? p : nullptr;
}

// activation input: device pointer used as is; host memory copied into the
// device staging area (counted as h2d traffic)
const void* stage_in(emelb_ctx* c, const void* p, uint64_t bytes, uint64_t slot_offset) {
  if (const void* d = resident_lookup(c, p)) return d;
  if (classify(c, p) == Where::device) return p;
  if (slot_offset + bytes > c->stage_in_bytes) return nullptr;
  void* d = static_cast<uint8_t*>(c->stage_in) + slot_offset;
  if (!cuda_ok(c, cudaMemcpyAsync(d, p, bytes, cudaMemcpyHostToDevice, c->stream))) return nullptr;
  c->diag.h2d_bytes += bytes;
  return d;
}

struct OutBinding {
  void* dev = nullptr;
  void* host = nullptr;
  uint64_t bytes = 0;
};

bool bind_out(emelb_ctx* c, const void* p, uint64_t bytes, uint64_t slot_offset, OutBinding* o) {
  o->bytes = bytes;
  if (classify(c, p) == Where::device) { o->dev = const_cast<void*>(p); return true; }
  if (slot_offset + bytes > c->stage_out_bytes) return false;
  o->dev = static_cast<uint8_t*>(c->stage_out) + slot_offset;
  o->host = const_cast<void*>(p);
  return true;
}

// copies a staged result back; the call then returns only after the bytes are
// in host memory (the reference's ops are synchronous)
bool finish_out(emelb_ctx* c, const OutBinding& o, bool* need_sync) {
  if (!o.host) return true;
  if (!cuda_ok(c, cudaMemcpyAsync(o.host, o.dev, o.bytes, cudaMemcpyDeviceToHost, c->stream))) return false;
  c->diag.d2h_bytes += o.bytes;
  *need_sync = true;
  return true;
}

uint32_t reject(emelb_ctx* c) {
  c->diag.rejected_dispatch_calls += 1;
  return EMELB_INVALID_REQUEST;
}

void count_dispatch(emelb_ctx* c, int type, uint64_t n, bool argmax) {
  switch (type) {
    case T_Q4_K: c->diag.optimized_q4_dispatch_calls += 1; if (n == 1) c->diag.optimized_q4_vector_dispatch_calls += 1; break;
    case T_Q6_K:
      c->diag.optimized_q6_dispatch_calls += 1;
      if (n == 1) c->diag.optimized_q6_vector_dispatch_calls += 1;
      if (argmax) c->diag.optimized_q6_vector_argmax_dispatch_calls += 1;
      break;
    case T_Q8_0: c->diag.optimized_q8_0_dispatch_calls += 1; break;
    case T_Q4_0: c->diag.optimized_q4_0_dispatch_calls += 1; break;
    default: break;
  }
}

}  // namespace

// ---- shared with the decoder (ctx.h)
namespace emelb {

thread_local bool g_pdl_launch = false;

ActPlanesMut ctx_planes(emelb_ctx* c) { return ActPlanesMut{c->act_qs, c->act_d, c->act_bsums}; }

ActPlanes planes_view(const ActPlanesMut& m, int type, int K) {
  ActPlanes a{};
  a.qs = m.qs;
  a.d = m.d;
  a.bsums = is_k_type(type) ? m.bsums : nullptr;
  a.col_stride_qs = K;
  a.col_stride_d = is_k_type(type) ? K / QK_K : K / QK32;
  a.col_stride_bs = K / 16;
  return a;
}

const void* ctx_resolve_weights(emelb_ctx* c, const void* p) { return resolve_weights(c, p); }
bool ctx_cuda_ok(emelb_ctx* c, cudaError_t e) { return cuda_ok(c, e); }

cudaError_t quantize_into_planes(int wtype, const float* x, int n, int ncols, int K, ActPlanesMut out, cudaStream_t st) {
  return is_k_type(wtype) ? launch_quantize_q8_k_planes(x, n, ncols, K, out, st)
                          : launch_quantize_q8_0_planes(x, n, ncols, K, out, st);
}

}  // namespace emelb

namespace emelb {
void comm_release(emelb_ctx* c);  // comm.cu
}

extern "C" {

uint32_t emelb_create(int device, emelb_ctx** out) {
  if (!out) return EMELB_INVALID_REQUEST;
  *out = nullptr;
  if (cudaSetDevice(device) != cudaSuccess) { cudaGetLastError(); return EMELB_INTERNAL_ERROR; }
  emelb_ctx* c = new (std::nothrow) emelb_ctx();
  if (!c) return EMELB_INTERNAL_ERROR;
  c->device = device;
  cudaDeviceProp prop{};
  if (cudaGetDeviceProperties(&prop, device) != cudaSuccess) { delete c; return EMELB_INTERNAL_ERROR; }
  c->sm_count = prop.multiProcessorCount;
  auto env_mb = [](const char* name, uint64_t def_mb) {
    const char* v = std::getenv(name);
    const uint64_t mb = v ? std::strtoull(v, nullptr, 10) : def_mb;
    return (mb ? mb : def_mb) << 20;
  };
  // EMELB_PDL=1: the decoder launches its kernel chain with programmatic stream serialization, so a
  // mat-vec starts prefetching weights while the kernel before it is still finishing
  c->pdl = std::getenv("EMELB_PDL") ? std::atoi(std::getenv("EMELB_PDL")) : 1;  // bit mask, see llama.cu
  c->stage_in_bytes = env_mb("EMELB_STAGE_IN_MB", 128);
  c->stage_out_bytes = env_mb("EMELB_STAGE_OUT_MB", 128);
  c->act_capacity = env_mb("EMELB_ACT_MELEMS", 64);  // quantized activation elements held at once
  bool ok = cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking) == cudaSuccess;
  ok = ok && cudaMalloc(&c->stage_in, c->stage_in_bytes) == cudaSuccess;
  ok = ok && cudaMalloc(&c->stage_out, c->stage_out_bytes) == cudaSuccess;
  ok = ok && cudaMalloc(&c->act_qs, c->act_capacity) == cudaSuccess;
  ok = ok && cudaMalloc(&c->act_d, c->act_capacity / 32 * sizeof(float)) == cudaSuccess;
  ok = ok && cudaMalloc(&c->act_bsums, c->act_capacity / 16 * sizeof(int16_t)) == cudaSuccess;
  // tiles of 128 columns x 256 K: 32 KB of int8 + 2.5 KB of block sums and scales; columns padded to 128
  c->tc_ws_bytes = c->act_capacity / 32768 * 35328 + (64u << 20);
  ok = ok && cudaMalloc(&c->tc_ws, c->tc_ws_bytes) == cudaSuccess;
  ok = ok && cudaMalloc(&c->gemv_sched, (2 * kSchedSlots + 2) * sizeof(int)) == cudaSuccess;
  ok = ok && cudaMemset(c->gemv_sched, 0, (2 * kSchedSlots + 2) * sizeof(int)) == cudaSuccess;
  c->bv_table_floats = 8u << 20;   // 32 MB: 57344 rows x 32 blocks (gate + up of the 70B shape) with room to spare
  c->grp_cnt_ints = 64u << 10;
  ok = ok && cudaMalloc(&c->bv_table, c->bv_table_floats * sizeof(float)) == cudaSuccess;
  ok = ok && cudaMalloc(&c->grp_cnt, c->grp_cnt_ints * sizeof(int)) == cudaSuccess;
  ok = ok && cudaMemset(c->grp_cnt, 0, c->grp_cnt_ints * sizeof(int)) == cudaSuccess;
  ok = ok && cudaMalloc(&c->token_bar, 4 * sizeof(unsigned)) == cudaSuccess;
  ok = ok && cudaMemset(c->token_bar, 0, 4 * sizeof(unsigned)) == cudaSuccess;
  ok = ok && cudaMalloc(&c->token_cnt, emelb_ctx::kTokenCounters * sizeof(int)) == cudaSuccess;
  ok = ok && cudaMemset(c->token_cnt, 0, emelb_ctx::kTokenCounters * sizeof(int)) == cudaSuccess;
  ok = ok && cudaMalloc(&c->part_val, kMaxArgmaxParts * sizeof(float)) == cudaSuccess;
  ok = ok && cudaMalloc(&c->part_idx, kMaxArgmaxParts * sizeof(int)) == cudaSuccess;
  ok = ok && cudaMalloc(&c->best_val, sizeof(float)) == cudaSuccess;
  ok = ok && cudaMalloc(&c->best_idx, sizeof(int)) == cudaSuccess;
  ok = ok && cudaMalloc(&c->fa_part_acc, kFlashPartFloats * sizeof(float)) == cudaSuccess;
  ok = ok && cudaMalloc(&c->fa_part_ml, kFlashPartFloats / 32 * sizeof(float)) == cudaSuccess;
  ok = ok && cudaMalloc(&c->fa_scores, kFlashScoreFloats * sizeof(float)) == cudaSuccess;
  if (!ok) {
    cudaGetLastError();
    emelb_destroy(c);
    return EMELB_INTERNAL_ERROR;
  }
  c->dev_ranges[reinterpret_cast<uintptr_t>(c->stage_in)] = c->stage_in_bytes;
  c->dev_ranges[reinterpret_cast<uintptr_t>(c->stage_out)] = c->stage_out_bytes;
  *out = c;
  return EMELB_OK;
}

uint32_t emelb_destroy(emelb_ctx* c) {
  if (!c) return EMELB_INVALID_REQUEST;
  cudaSetDevice(c->device);
  if (c->stream) cudaStreamSynchronize(c->stream);
  comm_release(c);
  upload_ring_release(c);
  for (auto& kv : c->residents)
    if (kv.second.dev) cudaFree(kv.second.dev);
  for (void* p : c->owned) cudaFree(p);
  void* bufs[] = {c->token_bar, c->token_cnt, c->bv_table, c->grp_cnt, c->gemv_sched, c->stage_in, c->stage_out, c->act_qs, c->act_d, c->act_bsums, c->tc_ws, c->part_val, c->part_idx,
                  c->best_val, c->best_idx, c->fa_part_acc, c->fa_part_ml, c->fa_scores};
  for (void* p : bufs)
    if (p) cudaFree(p);
  if (c->stream) cudaStreamDestroy(c->stream);
  cudaGetLastError();
  delete c;
  return EMELB_OK;
}

uint32_t emelb_sync(emelb_ctx* c) {
  if (!c) return EMELB_INVALID_REQUEST;
  if (!cuda_ok(c, cudaStreamSynchronize(c->stream))) return EMELB_INTERNAL_ERROR;
  // a kernel whose bounded wait ran out leaves 1 in the status word
  int status = 0;
  if (!cuda_ok(c, cudaMemcpy(&status, c->status_word(), sizeof(int), cudaMemcpyDeviceToHost))) return EMELB_INTERNAL_ERROR;
  if (status != 0) {
    // a kernel that gave up leaves task and arrival counters half-way
    cudaMemset(c->gemv_sched, 0, (2 * kSchedSlots + 2) * sizeof(int));
    cudaMemset(c->grp_cnt, 0, c->grp_cnt_ints * sizeof(int));
    cudaMemset(c->token_bar, 0, 4 * sizeof(unsigned));
    cudaMemset(c->token_cnt, 0, emelb_ctx::kTokenCounters * sizeof(int));
    return EMELB_INTERNAL_ERROR;
  }
  return EMELB_OK;
}

uint32_t emelb_get_stream(emelb_ctx* c, void** stream_out) {
  if (!c || !stream_out) return EMELB_INVALID_REQUEST;
  *stream_out = c->stream;
  return EMELB_OK;
}

uint32_t emelb_diagnostics(const emelb_ctx* c, emelb_diag* out) {
  if (!c || !out) return EMELB_INVALID_REQUEST;
  *out = c->diag;
  return EMELB_OK;
}

uint32_t emelb_set_upload_route(emelb_ctx* c, int32_t route, int32_t threads) {
  if (!c || route < EMELB_UPLOAD_RING || route > EMELB_UPLOAD_REGISTER || threads < 0) return EMELB_INVALID_REQUEST;
  c->upload_route = route;
  c->upload_threads = threads;
  return EMELB_OK;
}

uint32_t emelb_set_attention_mode(emelb_ctx* c, int mode) {
  if (!c || mode < 0 || mode > 2) return EMELB_INVALID_REQUEST;
  c->attention_mode = mode;
  return EMELB_OK;
}

// ------------------------------------------------------------------ residency
uint32_t emelb_residency_upload(emelb_ctx* c, int32_t tensor_id, const void* host, uint64_t bytes, int32_t tensor_type,
                                const void** dev_out) {
  UploadSpan span{tensor_id, host, bytes, tensor_type, 0, nullptr};
  const uint32_t err = emelb::residency_upload_many(c, &span, 1, -1);
  if (err == EMELB_OK && dev_out) *dev_out = span.dev;
  return err;
}

}  // extern "C"

uint32_t emelb::residency_upload_many(emelb_ctx* c, UploadSpan* spans, size_t count, int fd) {
  if (!c || !spans || count == 0) return EMELB_INVALID_REQUEST;
  for (size_t i = 0; i < count; ++i) {
    if (!spans[i].host || spans[i].bytes == 0) return EMELB_INVALID_REQUEST;
    auto found = c->residents.find(spans[i].tensor_id);
    if (found != c->residents.end() && found->second.state == EMELB_LIFECYCLE_RESIDENT) return EMELB_INVALID_REQUEST;
    for (size_t k = 0; k < i; ++k)
      if (spans[k].tensor_id == spans[i].tensor_id) return EMELB_INVALID_REQUEST;
  }
  cudaSetDevice(c->device);
  auto release = [&](size_t upto) {
    for (size_t k = 0; k < upto; ++k) {
      cudaFree(spans[k].dev);
      spans[k].dev = nullptr;
    }
  };
  for (size_t i = 0; i < count; ++i) {
    // padded so that 16-byte vector loads of the last row chunk stay inside the allocation
    if (!cuda_ok(c, cudaMalloc(&spans[i].dev, (spans[i].bytes + 255) & ~uint64_t(255)))) {
      release(i);
      c->residents[spans[i].tensor_id].state = EMELB_LIFECYCLE_INTERNAL_ERROR;
      return EMELB_INTERNAL_ERROR;
    }
  }
  if (!cuda_ok(c, upload_spans(c, spans, count, fd))) {
    release(count);
    return EMELB_INTERNAL_ERROR;
  }
  for (size_t i = 0; i < count; ++i) {
    Resident& r = c->residents[spans[i].tensor_id];
    if (r.host) c->by_host.erase(reinterpret_cast<uintptr_t>(r.host));
    r = Resident{EMELB_LIFECYCLE_RESIDENT, spans[i].dev, spans[i].bytes, spans[i].host, spans[i].tensor_type};
    c->by_host[reinterpret_cast<uintptr_t>(spans[i].host)] = spans[i].tensor_id;
    c->dev_ranges[reinterpret_cast<uintptr_t>(spans[i].dev)] = spans[i].bytes;
  }
  return EMELB_OK;
}

extern "C" {

uint32_t emelb_residency_evict(emelb_ctx* c, int32_t tensor_id) {
  if (!c) return EMELB_INVALID_REQUEST;
  auto it = c->residents.find(tensor_id);
  if (it == c->residents.end() || it->second.state != EMELB_LIFECYCLE_RESIDENT) return EMELB_INVALID_REQUEST;
  cudaStreamSynchronize(c->stream);
  cudaFree(it->second.dev);
  c->dev_ranges.erase(reinterpret_cast<uintptr_t>(it->second.dev));
  c->by_host.erase(reinterpret_cast<uintptr_t>(it->second.host));
  it->second.dev = nullptr;
  it->second.state = EMELB_LIFECYCLE_EVICTED;
  return EMELB_OK;
}

uint32_t emelb_residency_state(const emelb_ctx* c, int32_t tensor_id, emelb_tensor_state* out) {
  if (!c || !out) return EMELB_INVALID_REQUEST;
  auto it = c->residents.find(tensor_id);
  if (it == c->residents.end()) {
    *out = emelb_tensor_state{EMELB_LIFECYCLE_UNBOUND, nullptr, 0, nullptr, 0};
    return EMELB_OK;
  }
  const Resident& r = it->second;
  *out = emelb_tensor_state{(uint8_t)r.state, r.dev, r.bytes, r.host, r.type};
  return EMELB_OK;
}

uint32_t emelb_device_alloc(emelb_ctx* c, uint64_t bytes, void** dev_out) {
  if (!c || !dev_out || bytes == 0) return EMELB_INVALID_REQUEST;
  cudaSetDevice(c->device);
  void* p = nullptr;
  if (!cuda_ok(c, cudaMalloc(&p, (bytes + 255) & ~uint64_t(255)))) return EMELB_INTERNAL_ERROR;
  c->owned.insert(p);
  c->dev_ranges[reinterpret_cast<uintptr_t>(p)] = bytes;
  *dev_out = p;
  return EMELB_OK;
}

uint32_t emelb_device_free(emelb_ctx* c, void* dev) {
  if (!c || !c->owned.count(dev)) return EMELB_INVALID_REQUEST;
  cudaStreamSynchronize(c->stream);
  cudaFree(dev);
  c->owned.erase(dev);
  c->dev_ranges.erase(reinterpret_cast<uintptr_t>(dev));
  return EMELB_OK;
}

uint32_t emelb_copy_to_device(emelb_ctx* c, void* dev, const void* host, uint64_t bytes) {
  if (!c || !dev || !host) return EMELB_INVALID_REQUEST;
  const bool ok = cuda_ok(c, cudaMemcpyAsync(dev, host, bytes, cudaMemcpyHostToDevice, c->stream)) &&
                  cuda_ok(c, cudaStreamSynchronize(c->stream));
  return ok ? EMELB_OK : EMELB_INTERNAL_ERROR;
}

uint32_t emelb_copy_to_host(emelb_ctx* c, void* host, const void* dev, uint64_t bytes) {
  if (!c || !dev || !host) return EMELB_INVALID_REQUEST;
  const bool ok = cuda_ok(c, cudaMemcpyAsync(host, dev, bytes, cudaMemcpyDeviceToHost, c->stream)) &&
                  cuda_ok(c, cudaStreamSynchronize(c->stream));
  return ok ? EMELB_OK : EMELB_INTERNAL_ERROR;
}

// ------------------------------------------------------------------ guards
uint32_t emelb_can_run(const emelb_ctx* c, uint32_t op_code, const emelb_op* op) {
  (void)c;
  if (!op) return EMELB_INVALID_REQUEST;
  bool ok = false;
  if (op_code == EMELB_OP_MUL_MAT) ok = can_run_mul_mat(*op);
  else if (op_code == EMELB_OP_MUL_MAT_ARGMAX) ok = can_run_mul_mat_argmax(*op);
  else if (op_code == EMELB_OP_FLASH_ATTN_EXT) ok = can_run_flash(*op);
  else if (op_code == EMELB_OP_RMS_NORM) ok = can_run_rms_norm(*op);
  else if (op_code == EMELB_OP_ROPE) ok = can_run_rope(*op);
  else if (op_code == EMELB_OP_GLU) ok = false;   // no row executes op_glu in the reference's kernel actors either
  else return EMELB_UNSUPPORTED_OP;
  return ok ? EMELB_OK : EMELB_INVALID_REQUEST;
}

// ------------------------------------------------------------------ op_mul_mat
static uint32_t run_mul_mat(emelb_ctx* c, const emelb_op* op, bool argmax, bool prepared) {
  if (!c || !op) return EMELB_INVALID_REQUEST;
  if (!(argmax ? can_run_mul_mat_argmax(*op) : can_run_mul_mat(*op))) return reject(c);
  const int t = op->src0.type;
  // run_mul_mat_argmax has no Q4_0 branch (src/emel/kernel/detail.hpp:3621-3731)
  if (argmax && t == T_Q4_0) { c->diag.rejected_dispatch_calls += 1; return EMELB_UNSUPPORTED_OP; }
  const int K = (int)op->src0.ne[0], M = (int)op->src0.ne[1];
  const uint64_t n = op->src1.ne[0];
  cudaSetDevice(c->device);

  const bool preq = op->src1.type != T_F32;
  const uint64_t src1_bytes = preq ? row_bytes_of(op->src1.type, K) : n * (uint64_t)K * 4;
  // weights: resident span or device pointer; plain host weights (never uploaded)
  // are copied through the staging area behind src1 on every call
  const uint8_t* W = static_cast<const uint8_t*>(resolve_weights(c, op->src0.data));
  if (!W) {
    W = static_cast<const uint8_t*>(stage_in(c, op->src0.data, (uint64_t)M * op->src0.nb[1], (src1_bytes + 255) & ~uint64_t(255)));
    if (!W) { c->diag.rejected_dispatch_calls += 1; return EMELB_UNSUPPORTED_OP; }
  }
  const void* x = nullptr;
  if (prepared) {
    // the planes left by emelb_prepare_rhs must describe this src1
    if (preq || c->prepared_n != n || c->prepared_k != (uint64_t)K || c->prepared_k_family != is_k_type(t)) return reject(c);
  } else {
    c->prepared_n = 0;  // the planes are about to be overwritten
    x = stage_in(c, op->src1.data, src1_bytes, 0);
    if (!x) { c->diag.rejected_dispatch_calls += 1; return EMELB_UNSUPPORTED_OP; }
  }

  // argmax writes the context's result cells, copied out at the end
  OutBinding out{};
  if (!argmax && !bind_out(c, op->dst.data, n * (uint64_t)M * 4, 0, &out)) {
    c->diag.rejected_dispatch_calls += 1;
    return EMELB_UNSUPPORTED_OP;
  }

  int launches = 0;
  const ActPlanesMut planes = ctx_planes(c);
  GemvArgs a{};
  a.W = W;
  a.row_bytes = (int64_t)op->src0.nb[1];
  a.M = M;
  a.K = K;
  a.act = planes_view(planes, t, K);
  a.y = static_cast<float*>(out.dev);
  a.ldy = (int64_t)n;
  a.residual = nullptr;
  a.tc_ws = c->tc_ws;
  a.tc_ws_bytes = c->tc_ws_bytes;
  // streaming mat-vec launches carry the programmatic-serialization attribute: the kernel starts its weight
  // copies while the previous kernel of the stream drains and waits (griddepcontrol.wait) before it reads
  // activations or writes results, so stream order is kept
  a.pdl = c->pdl & 1;
  a.sched = c->next_sched();
  a.status = c->status_word();
  a.part_val = c->part_val;
  a.part_idx = c->part_idx;
  a.best_val = c->best_val;
  a.best_idx = c->best_idx;

  bool ok = true;
  if (prepared) {
    a.col0 = 0;
    ok = cuda_ok(c, launch_gemv(t, a, (int)n, argmax, c->sm_count, c->stream, &launches));
  } else if (preq) {
    ok = cuda_ok(c, launch_blocks_to_planes(op->src1.type, static_cast<const uint8_t*>(x), K, planes, c->stream));
    ++launches;
    a.col0 = 0;
    ok = ok && cuda_ok(c, launch_gemv(t, a, 1, false, c->sm_count, c->stream, &launches));
  } else {
    // columns are quantized in tiles that fit the activation planes
    const uint64_t tile = c->act_capacity / (uint64_t)K ? c->act_capacity / (uint64_t)K : 1;
    for (uint64_t j0 = 0; ok && j0 < n; j0 += tile) {
      const int cols = (int)((n - j0) < tile ? (n - j0) : tile);
      // column j of src1 is x[p*n + j]: a tile starts j0 floats in, same stride n
      ok = cuda_ok(c, quantize_into_planes(t, static_cast<const float*>(x) + j0, (int)n, cols, K, planes, c->stream));
      ++launches;
      GemvArgs b = a;
      b.sched = c->next_sched();
      b.col0 = 0;
      b.y = a.y + j0;
      if (argmax) b.y = nullptr;
      ok = ok && cuda_ok(c, launch_gemv(t, b, cols, argmax, c->sm_count, c->stream, &launches));
    }
  }
  c->diag.kernel_launches += launches;
  if (!ok) return EMELB_INTERNAL_ERROR;
  count_dispatch(c, t, n, argmax);

  bool need_sync = false;
  if (argmax) {
    const Where wd = classify(c, op->dst.data), wi = classify(c, op->index_out);
    ok = cuda_ok(c, cudaMemcpyAsync(const_cast<void*>(op->dst.data), c->best_val, 4,
                                    wd == Where::device ? cudaMemcpyDeviceToDevice : cudaMemcpyDeviceToHost, c->stream));
    ok = ok && cuda_ok(c, cudaMemcpyAsync(op->index_out, c->best_idx, 4,
                                          wi == Where::device ? cudaMemcpyDeviceToDevice : cudaMemcpyDeviceToHost, c->stream));
    if (wd != Where::device) c->diag.d2h_bytes += 4;
    if (wi != Where::device) c->diag.d2h_bytes += 4;
    need_sync = wd != Where::device || wi != Where::device;
  } else {
    ok = finish_out(c, out, &need_sync);
  }
  if (ok && need_sync) ok = cuda_ok(c, cudaStreamSynchronize(c->stream));
  return ok ? EMELB_OK : EMELB_INTERNAL_ERROR;
}

uint32_t emelb_mul_mat(emelb_ctx* c, const emelb_op* op) { return run_mul_mat(c, op, false, false); }
uint32_t emelb_mul_mat_argmax(emelb_ctx* c, const emelb_op* op) { return run_mul_mat(c, op, true, false); }
uint32_t emelb_mul_mat_prepared(emelb_ctx* c, const emelb_op* op) { return run_mul_mat(c, op, false, true); }

// two or three products against the same prepared column in one launch (what the decoder does for Q, K, V and
// for gate, up); anything the grouped launch does not take runs as `count` single products, same results
uint32_t emelb_mul_mat_prepared_group(emelb_ctx* c, const emelb_op* ops, uint32_t count) {
  if (!c || !ops || count == 0) return EMELB_INVALID_REQUEST;
  bool group = count >= 2 && count <= 3;
  const uint8_t* W[3] = {nullptr, nullptr, nullptr};
  for (uint32_t i = 0; group && i < count; ++i) {
    const emelb_op& o = ops[i];
    group = can_run_mul_mat(o) && o.src1.type == T_F32 && o.src1.ne[0] == 1 && o.src0.type == ops[0].src0.type &&
            o.src0.ne[0] == ops[0].src0.ne[0] && o.src0.nb[1] == ops[0].src0.nb[1] && c->prepared_n == 1 &&
            c->prepared_k == o.src0.ne[0] && c->prepared_k_family == is_k_type(o.src0.type) &&
            classify(c, o.dst.data) == Where::device;
    if (group) W[i] = static_cast<const uint8_t*>(resolve_weights(c, o.src0.data));
    group = group && W[i] && gemv_fast_path_ok(o.src0.type, W[i], (int64_t)o.src0.nb[1], (int)o.src0.ne[0]);
  }
  if (!group) {
    for (uint32_t i = 0; i < count; ++i) {
      const uint32_t err = run_mul_mat(c, &ops[i], false, true);
      if (err != EMELB_OK) return err;
    }
    return EMELB_OK;
  }
  cudaSetDevice(c->device);
  const int t = ops[0].src0.type, K = (int)ops[0].src0.ne[0];
  GemvArgs a{};
  a.W = W[0];
  a.row_bytes = (int64_t)ops[0].src0.nb[1];
  a.M = (int)ops[0].src0.ne[1];
  a.K = K;
  a.act = planes_view(ctx_planes(c), t, K);
  a.y = static_cast<float*>(const_cast<void*>(ops[0].dst.data));
  a.ldy = 1;
  a.W2 = W[1];
  a.M2 = (int)ops[1].src0.ne[1];
  a.y2 = static_cast<float*>(const_cast<void*>(ops[1].dst.data));
  if (count == 3) {
    a.W3 = W[2];
    a.M3 = (int)ops[2].src0.ne[1];
    a.y3 = static_cast<float*>(const_cast<void*>(ops[2].dst.data));
  }
  a.pdl = c->pdl & 1;
  a.sched = c->next_sched();
  a.status = c->status_word();
  int launches = 0;
  if (!cuda_ok(c, launch_gemv(t, a, 1, false, c->sm_count, c->stream, &launches))) return EMELB_INTERNAL_ERROR;
  c->diag.kernel_launches += launches;
  for (uint32_t i = 0; i < count; ++i) count_dispatch(c, t, 1, false);
  return EMELB_OK;
}

uint32_t emelb_prepare_rhs(emelb_ctx* c, const emelb_view* src1, int32_t weight_type) {
  if (!c || !src1 || !src1->data) return EMELB_INVALID_REQUEST;
  const uint64_t n = src1->ne[0], K = src1->ne[1];
  const uint64_t be = block_elems(weight_type);
  const uint64_t lim = is_32_type(weight_type) ? MAX_Q8_0_BLOCKS : MAX_Q8_K_BLOCKS;
  if (!is_native_quant(weight_type) || src1->type != T_F32 || !dense(*src1) || n == 0 || K == 0 || K % be != 0 ||
      K / be > lim || src1->ne[2] != 1 || src1->ne[3] != 1 || n * K > c->act_capacity)
    return reject(c);
  cudaSetDevice(c->device);
  c->prepared_n = 0;
  const void* x = stage_in(c, src1->data, n * K * 4, 0);
  if (!x) { c->diag.rejected_dispatch_calls += 1; return EMELB_UNSUPPORTED_OP; }
  if (!cuda_ok(c, quantize_into_planes(weight_type, static_cast<const float*>(x), (int)n, (int)n, (int)K, ctx_planes(c), c->stream)))
    return EMELB_INTERNAL_ERROR;
  c->diag.kernel_launches += 1;
  c->prepared_n = n;
  c->prepared_k = K;
  c->prepared_k_family = is_k_type(weight_type);
  return EMELB_OK;
}

// ------------------------------------------------------------------ attention over a token batch
uint32_t emelb_flash_attn_batch(emelb_ctx* c, const float* q, const void* k, const void* v, float* dst, int32_t head_dim,
                                int32_t heads, int32_t kv_heads, int32_t batch, int32_t pos0, int64_t cache_head_stride,
                                float scale) {
  if (!c) return EMELB_INVALID_REQUEST;
  if (!q || !k || !v || !dst || batch <= 0 || pos0 < 0 || heads <= 0 || kv_heads <= 0 || head_dim <= 0 ||
      cache_head_stride < (int64_t)(pos0 + batch) * head_dim)
    return reject(c);
  for (const void* p : {(const void*)q, k, v, (const void*)dst})
    if (classify(c, p) != Where::device) return reject(c);
  cudaSetDevice(c->device);
  PrefillAttnArgs a{q, dst, static_cast<const __half*>(k), static_cast<const __half*>(v), cache_head_stride,
                    head_dim, heads, kv_heads, batch, pos0, scale};
  if (!prefill_attention_supported(a)) {
    c->diag.rejected_dispatch_calls += 1;
    return EMELB_UNSUPPORTED_OP;
  }
  if (!cuda_ok(c, launch_prefill_attention(a, c->stream))) return EMELB_INTERNAL_ERROR;
  c->diag.kernel_launches += 1;
  c->diag.optimized_flash_dispatch_calls += 1;
  return EMELB_OK;
}

// ------------------------------------------------------------------ op_flash_attn_ext
uint32_t emelb_flash_attn_ext(emelb_ctx* c, const emelb_op* op) {
  if (!c || !op) return EMELB_INVALID_REQUEST;
  if (!can_run_flash(*op)) return reject(c);
  cudaSetDevice(c->device);
  const int D = (int)op->src0.ne[0], H = (int)op->src0.ne[2], T = (int)op->src1.ne[1], Hkv = (int)op->src1.ne[2];
  auto span = [&](const emelb_view& v) { return (uint64_t)(Hkv - 1) * v.nb[2] + (uint64_t)(T - 1) * v.nb[1] + (uint64_t)D * 2; };
  const uint64_t qbytes = (uint64_t)D * H * 4;
  const uint64_t kspan = span(op->src1), vspan = span(op->src2);
  const uint64_t koff = (qbytes + 255) & ~uint64_t(255);
  const uint64_t voff = (koff + kspan + 255) & ~uint64_t(255);
  const void* q = stage_in(c, op->src0.data, qbytes, 0);
  const void* k = stage_in(c, op->src1.data, kspan, koff);
  const void* v = stage_in(c, op->src2.data, vspan, voff);
  OutBinding out{};
  if (!q || !k || !v || !bind_out(c, op->dst.data, qbytes, 0, &out)) {
    c->diag.rejected_dispatch_calls += 1;
    return EMELB_UNSUPPORTED_OP;
  }
  FlashArgs a{};
  a.q = static_cast<const float*>(q);
  a.k = static_cast<const __half*>(k);
  a.v = static_cast<const __half*>(v);
  a.dst = static_cast<float*>(out.dev);
  a.k_nb1 = (int64_t)op->src1.nb[1]; a.k_nb2 = (int64_t)op->src1.nb[2];
  a.v_nb1 = (int64_t)op->src2.nb[1]; a.v_nb2 = (int64_t)op->src2.nb[2];
  a.head_dim = D; a.heads = H; a.kv_heads = Hkv; a.tokens = T; a.tokens_dev = nullptr;
  a.scale = fa_scale(*op);
  a.part_acc = c->fa_part_acc;
  a.part_ml = c->fa_part_ml;
  int max_splits = (int)(kFlashPartFloats / ((uint64_t)H * D));
  if (max_splits > 64) max_splits = 64;
  a.splits = max_splits >= 1 ? flash_pick_splits(T, Hkv, c->sm_count, max_splits) : 0;

  int launches = 0;
  bool ok;
  const bool fast = c->attention_mode == 0 && a.splits >= 1 && flash_split_supported(a);
  if (fast) {
    ok = cuda_ok(c, launch_flash_decode(a, c->sm_count, c->stream, &launches, 0, ActPlanesMut{}));
    c->diag.optimized_flash_dispatch_calls += 1;
  } else {
    if ((uint64_t)H * (uint64_t)T > kFlashScoreFloats) { c->diag.rejected_dispatch_calls += 1; return EMELB_UNSUPPORTED_OP; }
    ok = cuda_ok(c, launch_flash_reference_order(a, c->fa_scores, T, c->attention_mode == 1 ? 1 : 2, c->stream, &launches));
    c->diag.shared_flash_dispatch_calls += 1;
  }
  c->diag.kernel_launches += launches;
  bool need_sync = false;
  ok = ok && finish_out(c, out, &need_sync);
  if (ok && need_sync) ok = cuda_ok(c, cudaStreamSynchronize(c->stream));
  return ok ? EMELB_OK : EMELB_INTERNAL_ERROR;
}

// ------------------------------------------------------------------ op_rms_norm / op_rope
namespace {

// bytes from the first to one past the last element of a strided f32 / i32 tensor
uint64_t covering_span(const emelb_view& v) {
  uint64_t span = 4;
  for (int i = 0; i < 4; ++i) span += (v.ne[i] - 1) * stride_bytes(v, i);
  return span;
}
StridedF32 strided(const emelb_view& v, void* dev) {
  StridedF32 s{};
  s.base = static_cast<char*>(dev);
  for (int i = 0; i < 4; ++i) {
    s.ne[i] = (int64_t)v.ne[i];
    s.nb[i] = (int64_t)stride_bytes(v, i);
  }
  return s;
}
// a host destination whose elements do not fill its covering span is staged in first, so that the bytes between
// the elements go back unchanged
bool bind_strided_out(emelb_ctx* c, const emelb_view& v, OutBinding* o) {
  const uint64_t span = covering_span(v);
  if (!bind_out(c, v.data, span, 0, o)) return false;
  if (o->host && !dense(v)) {
    if (!cuda_ok(c, cudaMemcpyAsync(o->dev, o->host, span, cudaMemcpyHostToDevice, c->stream))) return false;
    c->diag.h2d_bytes += span;
  }
  return true;
}

}  // namespace

uint32_t emelb_rms_norm(emelb_ctx* c, const emelb_op* op) {
  if (!c || !op) return EMELB_INVALID_REQUEST;
  if (!can_run_rms_norm(*op)) return reject(c);
  cudaSetDevice(c->device);
  float eps = 0.0f;
  read_param_f32(*op, 0, &eps);
  const void* x = stage_in(c, op->src0.data, covering_span(op->src0), 0);
  OutBinding out{};
  if (!x || !bind_strided_out(c, op->dst, &out)) {
    c->diag.rejected_dispatch_calls += 1;
    return EMELB_UNSUPPORTED_OP;
  }
  bool ok = cuda_ok(c, launch_rms_norm_rows(strided(op->src0, const_cast<void*>(x)), strided(op->dst, out.dev), eps, c->stream));
  c->diag.kernel_launches += 1;
  bool need_sync = false;
  ok = ok && finish_out(c, out, &need_sync);
  if (ok && need_sync) ok = cuda_ok(c, cudaStreamSynchronize(c->stream));
  return ok ? EMELB_OK : EMELB_INTERNAL_ERROR;
}

uint32_t emelb_rope(emelb_ctx* c, const emelb_op* op) {
  if (!c || !op) return EMELB_INVALID_REQUEST;
  if (!can_run_rope(*op)) return reject(c);
  RopeParams p;
  read_rope_params(*op, &p);
  // the adjacent-pair and the half-split pairing; the reference's third variant (mode 4, a timestep embedding with
  // its own layout) is not on this path
  if (p.mode != kRopeNorm && p.mode != kRopeNeox) { c->diag.rejected_dispatch_calls += 1; return EMELB_UNSUPPORTED_OP; }
  cudaSetDevice(c->device);
  const uint64_t xspan = covering_span(op->src0);
  const uint64_t poff = (xspan + 255) & ~uint64_t(255);
  const void* x = stage_in(c, op->src0.data, xspan, 0);
  const void* pos = stage_in(c, op->src1.data, covering_span(op->src1), poff);
  OutBinding out{};
  if (!x || !pos || !bind_strided_out(c, op->dst, &out)) {
    c->diag.rejected_dispatch_calls += 1;
    return EMELB_UNSUPPORTED_OP;
  }
  // std::pow(freq_base, -2.0f / n_dims) with the host's libm, as the reference computes it: the angles are then
  // the reference's floats bit for bit (the device's cosf / sinf differ from the host's in the last place at most)
  const float theta_scale = ::powf(p.freq_base, -2.0f / (float)p.n_dims);
  bool ok = cuda_ok(c, launch_rope_rows(strided(op->src0, const_cast<void*>(x)), strided(op->dst, out.dev), static_cast<const char*>(pos),
                                        (int64_t)stride_bytes(op->src1, 0), p.n_dims, p.mode == kRopeNeox ? 1 : 0, theta_scale,
                                        p.freq_scale, p.attn_factor, c->stream));
  c->diag.kernel_launches += 1;
  bool need_sync = false;
  ok = ok && finish_out(c, out, &need_sync);
  if (ok && need_sync) ok = cuda_ok(c, cudaStreamSynchronize(c->stream));
  return ok ? EMELB_OK : EMELB_INTERNAL_ERROR;
}

uint32_t emelb_glu(emelb_ctx* c, const emelb_op* op) {
  // every op_glu request is rejected by the reference's kernel actors (can_run_backend_request falls through to
  // can_execute_scalar, which has no op_glu branch: src/emel/kernel/detail.hpp:5166-5203, 5315-5335); the SwiGLU
  // of the decoder layer is the generator's own loop, restated inside emelb_llama
  if (!c || !op) return EMELB_INVALID_REQUEST;
  return reject(c);
}

// ------------------------------------------------------------------ kernel::attention head-range event
namespace {
bool ranges_disjoint(const void* a, uint64_t a_bytes, const void* b, uint64_t b_bytes) {
  const uintptr_t ab = reinterpret_cast<uintptr_t>(a), bb = reinterpret_cast<uintptr_t>(b);
  if (ab > UINTPTR_MAX - a_bytes || bb > UINTPTR_MAX - b_bytes) return false;
  return ab + a_bytes <= bb || bb + b_bytes <= ab;
}
// guard_request_shape_supported (src/emel/kernel/attention/guards.hpp:28-90)
bool head_range_ok(const emelb_head_range_request& r) {
  if (r.hidden_dim <= 0 || r.head_dim <= 0 || r.head_begin < 0 || r.head_end <= r.head_begin || r.position_capacity <= 0 ||
      r.physical_begin < 0 || r.physical_begin >= r.position_capacity || r.valid_positions <= 0 ||
      r.valid_positions > r.position_capacity)
    return false;
  const uint64_t hidden = (uint64_t)r.hidden_dim, hd = (uint64_t)r.head_dim, cap = (uint64_t)r.position_capacity;
  const uint64_t heads = (uint64_t)(r.head_end - r.head_begin), mx = UINT64_MAX;
  if (cap > (mx - r.layer_offset) / hidden || heads > mx / hd || (uint64_t)r.head_end > hidden / hd) return false;
  const uint64_t cache_required = r.layer_offset + cap * hidden, output_required = heads * hd;
  if (hd > 8192 || cap > 8192 || !r.query || !r.key_cache || !r.value_cache || !r.output || r.query_count < hidden ||
      r.key_count < cache_required || r.value_count < cache_required || r.output_count < output_required ||
      reinterpret_cast<uintptr_t>(r.query) % alignof(float) != 0 || reinterpret_cast<uintptr_t>(r.key_cache) % alignof(uint16_t) != 0 ||
      reinterpret_cast<uintptr_t>(r.value_cache) % alignof(uint16_t) != 0 || reinterpret_cast<uintptr_t>(r.output) % alignof(float) != 0 ||
      hidden > mx / sizeof(float) || cache_required > mx / sizeof(uint16_t) || output_required > mx / sizeof(float))
    return false;
  const uint64_t qb = hidden * sizeof(float), cb = cache_required * sizeof(uint16_t), ob = output_required * sizeof(float);
  return ranges_disjoint(r.output, ob, r.query, qb) && ranges_disjoint(r.output, ob, r.key_cache, cb) &&
         ranges_disjoint(r.output, ob, r.value_cache, cb);
}
}  // namespace

uint32_t emelb_attention_head_range_can_run(const emelb_head_range_request* r) {
  return r && head_range_ok(*r) ? EMELB_OK : EMELB_INVALID_REQUEST;
}

uint32_t emelb_attention_head_range(emelb_ctx* c, const emelb_head_range_request* r) {
  if (!c || !r) return EMELB_INVALID_REQUEST;
  if (!head_range_ok(*r)) return reject(c);
  cudaSetDevice(c->device);
  const uint64_t hidden = (uint64_t)r->hidden_dim, cache_elems = r->layer_offset + (uint64_t)r->position_capacity * hidden;
  const uint64_t qb = hidden * 4, cb = cache_elems * 2, ob = (uint64_t)(r->head_end - r->head_begin) * r->head_dim * 4;
  auto up = [](uint64_t b) { return (b + 255) & ~uint64_t(255); };
  const void* q = stage_in(c, r->query, qb, 0);
  const void* k = stage_in(c, r->key_cache, cb, up(qb));
  const void* v = stage_in(c, r->value_cache, cb, up(qb) + up(cb));
  OutBinding out{};
  if (!q || !k || !v || !bind_out(c, r->output, ob, 0, &out)) {
    c->diag.rejected_dispatch_calls += 1;
    return EMELB_UNSUPPORTED_OP;   // host caches larger than the staging area
  }
  HeadRangeArgs a{};
  a.query = static_cast<const float*>(q);
  a.key = static_cast<const uint16_t*>(k);
  a.value = static_cast<const uint16_t*>(v);
  a.output = static_cast<float*>(out.dev);
  a.layer_offset = (size_t)r->layer_offset;
  a.hidden_dim = r->hidden_dim;
  a.head_dim = r->head_dim;
  a.head_begin = r->head_begin;
  a.head_end = r->head_end;
  a.capacity = r->position_capacity;
  a.physical_begin = r->physical_begin;
  a.valid = r->valid_positions;
  a.scale = 1.0f / std::sqrt((float)r->head_dim);
  bool ok = cuda_ok(c, launch_head_range_attention(a, c->stream));
  c->diag.kernel_launches += 1;
  bool need_sync = false;
  ok = ok && finish_out(c, out, &need_sync);
  if (ok && need_sync) ok = cuda_ok(c, cudaStreamSynchronize(c->stream));
  return ok ? EMELB_OK : EMELB_INTERNAL_ERROR;
}

// ------------------------------------------------------------------ quantize / dequantize
uint32_t emelb_quantize(emelb_ctx* c, const emelb_view* src, const emelb_view* dst) {
  if (!c || !src || !dst || !src->data || !dst->data) return EMELB_INVALID_REQUEST;
  const int t = dst->type;
  if (src->type != T_F32 || (t != T_Q8_K && t != T_Q8_0) || !dense(*src)) return reject(c);
  const uint64_t n = src->ne[0], K = src->ne[1];
  const uint64_t rb = row_bytes_of(t, K);
  const uint64_t lim = t == T_Q8_K ? MAX_Q8_K_BLOCKS : MAX_Q8_0_BLOCKS;
  if (n == 0 || K == 0 || rb == 0 || K / block_elems(t) > lim || dst->ne[0] != K || dst->ne[1] != n || dst->nb[1] < rb ||
      dst->nb[1] % (t == T_Q8_K ? 4 : 2) != 0 || src->ne[2] != 1 || src->ne[3] != 1)
    return reject(c);
  cudaSetDevice(c->device);
  const void* x = stage_in(c, src->data, n * K * 4, 0);
  OutBinding out{};
  if (!x || !bind_out(c, dst->data, (n - 1) * dst->nb[1] + rb, 0, &out)) {
    c->diag.rejected_dispatch_calls += 1;
    return EMELB_UNSUPPORTED_OP;
  }
  bool ok = cuda_ok(c, t == T_Q8_K ? launch_quantize_q8_k_blocks(static_cast<const float*>(x), (int)n, (int)K,
                                                                 static_cast<uint8_t*>(out.dev), (int64_t)dst->nb[1], c->stream)
                                   : launch_quantize_q8_0_blocks(static_cast<const float*>(x), (int)n, (int)K,
                                                                 static_cast<uint8_t*>(out.dev), (int64_t)dst->nb[1], c->stream));
  c->diag.kernel_launches += 1;
  bool need_sync = false;
  ok = ok && finish_out(c, out, &need_sync);
  if (ok && need_sync) ok = cuda_ok(c, cudaStreamSynchronize(c->stream));
  return ok ? EMELB_OK : EMELB_INTERNAL_ERROR;
}

uint32_t emelb_dequantize(emelb_ctx* c, const emelb_view* src, const emelb_view* dst) {
  if (!c || !src || !dst || !dst->data) return EMELB_INVALID_REQUEST;
  if (!required_src0_matmul(*src) || !is_native_quant(src->type) || dst->type != T_F32 || !dense(*dst) ||
      dst->ne[0] != src->ne[0] || dst->ne[1] != src->ne[1] || dst->ne[2] != 1 || dst->ne[3] != 1)
    return reject(c);
  cudaSetDevice(c->device);
  const uint64_t K = src->ne[0], M = src->ne[1];
  const void* w = resident_lookup(c, src->data);
  if (!w) w = stage_in(c, src->data, M * src->nb[1], 0);
  OutBinding out{};
  if (!w || !bind_out(c, dst->data, K * M * 4, 0, &out)) {
    c->diag.rejected_dispatch_calls += 1;
    return EMELB_UNSUPPORTED_OP;
  }
  bool ok = cuda_ok(c, launch_dequantize(src->type, static_cast<const uint8_t*>(w), (int64_t)src->nb[1],
                                         static_cast<float*>(out.dev), (int64_t)K, (int)K, (int)M, c->stream));
  c->diag.kernel_launches += 1;
  bool need_sync = false;
  ok = ok && finish_out(c, out, &need_sync);
  if (ok && need_sync) ok = cuda_ok(c, cudaStreamSynchronize(c->stream));
  return ok ? EMELB_OK : EMELB_INTERNAL_ERROR;
}

// ------------------------------------------------------------------ graphs
uint32_t emelb_graph_begin(emelb_ctx* c) {
  if (!c || c->capturing) return EMELB_INVALID_REQUEST;
  cudaSetDevice(c->device);
  if (!cuda_ok(c, cudaStreamBeginCapture(c->stream, cudaStreamCaptureModeThreadLocal))) return EMELB_INTERNAL_ERROR;
  c->capturing = true;
  return EMELB_OK;
}

uint32_t emelb_graph_end(emelb_ctx* c, void** graph_out) {
  if (!c || !graph_out || !c->capturing) return EMELB_INVALID_REQUEST;
  c->capturing = false;
  cudaGraph_t g = nullptr;
  if (!cuda_ok(c, cudaStreamEndCapture(c->stream, &g)) || !g) return EMELB_INTERNAL_ERROR;
  cudaGraphExec_t ex = nullptr;
  const bool ok = cuda_ok(c, cudaGraphInstantiate(&ex, g, 0));
  cudaGraphDestroy(g);
  if (!ok) return EMELB_INTERNAL_ERROR;
  *graph_out = ex;
  return EMELB_OK;
}

uint32_t emelb_graph_launch(emelb_ctx* c, void* graph) {
  if (!c || !graph || c->capturing) return EMELB_INVALID_REQUEST;
  return cuda_ok(c, cudaGraphLaunch(static_cast<cudaGraphExec_t>(graph), c->stream)) ? EMELB_OK : EMELB_INTERNAL_ERROR;
}

uint32_t emelb_graph_destroy(emelb_ctx* c, void* graph) {
  if (!c || !graph) return EMELB_INVALID_REQUEST;
  cudaStreamSynchronize(c->stream);
  return cuda_ok(c, cudaGraphExecDestroy(static_cast<cudaGraphExec_t>(graph))) ? EMELB_OK : EMELB_INTERNAL_ERROR;
}

// ------------------------------------------------------------------ synthetic data
uint32_t emelb_synth_fill(emelb_ctx* c, void* dev, int32_t type, uint64_t elems, uint64_t seed, float sigma, uint64_t offset) {
  if (!c || !dev || elems == 0) return EMELB_INVALID_REQUEST;
  cudaSetDevice(c->device);
  cudaError_t e;
  if (type == T_F32) e = launch_fill_normal(static_cast<float*>(dev), elems, seed, sigma, offset, c->stream);
  else if (is_native_quant(type) && elems % block_elems(type) == 0)
    e = launch_encode_normal(type, static_cast<uint8_t*>(dev), elems, seed, sigma, offset, c->stream);
  else return EMELB_INVALID_REQUEST;
  c->diag.kernel_launches += 1;
  return cuda_ok(c, e) ? EMELB_OK : EMELB_INTERNAL_ERROR;
}

// ------------------------------------------------------------------ row slices
uint32_t emelb_row_slice(const emelb_op* op, uint32_t lane, uint32_t lane_count, emelb_op* out, uint64_t* row_begin,
                         uint64_t* row_count) {
  if (!op || !out || lane_count == 0 || lane >= lane_count) return EMELB_INVALID_REQUEST;
  const uint64_t rows = op->src0.ne[1];
  const uint64_t per = rows / lane_count, extra = rows % lane_count;
  const uint64_t begin = lane * per + (lane < extra ? lane : extra);
  const uint64_t count = per + (lane < extra ? 1u : 0u);
  *out = *op;
  out->src0.data = static_cast<const uint8_t*>(op->src0.data) + begin * op->src0.nb[1];
  out->src0.ne[1] = count;
  out->src0.nb[2] = op->src0.nb[1] * count;
  out->src0.nb[3] = out->src0.nb[2];
  out->dst.data = static_cast<const uint8_t*>(op->dst.data) + begin * op->dst.nb[1];
  out->dst.ne[1] = count;
  out->dst.nb[2] = op->dst.nb[1] * count;
  out->dst.nb[3] = out->dst.nb[2];
  if (row_begin) *row_begin = begin;
  if (row_count) *row_count = count;
  return EMELB_OK;
}

}  // extern "C"
