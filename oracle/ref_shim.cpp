// TEST INFRASTRUCTURE ONLY — never linked into or called by the product path.
//
// Thin extern "C" exports over the reference's own kernel headers, included in
// place from the reference checkout (-I<reference>/src -I<reference>/include;
// nothing is copied).  Built into oracle/_ref/libemel_ref.so by
// oracle/Makefile with `g++ -O2 -std=c++20 -ffp-contract=off` and no global
// -mavx2/-mfma: the AVX2 functions carry their own target attributes
// (src/emel/kernel/x86_64/actions.hpp:22-37), and contraction is off so that
// "bit-exact against the reference" names one well-defined build.
//
// Uses: validating oracle/emel_oracle.c, generating tests/golden fixtures,
// being the checker in the GPU parity tests, and the timed CPU baseline.

#include <cstdint>
#include <cstring>
#include <thread>
#include <vector>

#include "emel/gguf/loader/detail.hpp"
#include "emel/kernel/attention/actions.hpp"
#include "emel/kernel/attention/guards.hpp"
#include "emel/kernel/x86_64/actions.hpp"

#include "../include/emelb.h"

namespace kd = ::emel::kernel::detail;
namespace kq = ::emel::kernel::detail::quant;
namespace kx = ::emel::kernel::x86_64::detail;
namespace ev = ::emel::kernel::event;

namespace {

ev::tensor_view to_view(const emelb_view& v) {
  ev::tensor_view out{};
  out.data = v.data;
  out.type = static_cast<ev::dtype>(v.type);
  for (int i = 0; i < 4; ++i) {
    out.ne[i] = v.ne[i];
    out.nb[i] = v.nb[i];
  }
  return out;
}

ev::tensor_view_mut to_view_mut(const emelb_view& v) {
  ev::tensor_view_mut out{};
  out.data = const_cast<void*>(v.data);
  out.type = static_cast<ev::dtype>(v.type);
  for (int i = 0; i < 4; ++i) {
    out.ne[i] = v.ne[i];
    out.nb[i] = v.nb[i];
  }
  return out;
}

template <class op_type>
op_type to_op(const emelb_op& op) {
  op_type out{};
  out.src0 = to_view(op.src0);
  out.src1 = to_view(op.src1);
  out.src2 = to_view(op.src2);
  out.dst = to_view_mut(op.dst);
  std::memcpy(out.op_params.data(), op.op_params, 64);
  out.op_params_size = op.op_params_size;
  return out;
}

}  // namespace

extern "C" {

// ---- fp16 <-> fp32 (src/emel/kernel/detail.hpp:350-392)
float ref_fp16_to_fp32(uint16_t h) { return kq::fp16_to_fp32(h); }
uint16_t ref_fp32_to_fp16(float f) { return kq::fp32_to_fp16(f); }

// ---- activation quantizers (src/emel/kernel/detail.hpp:804-867)
void ref_quantize_q8_k(const float* x, uint64_t stride, void* y, int64_t k) {
  kq::quantize_row_q8_k_strided(x, stride, static_cast<kq::block_q8_k*>(y), k);
}
void ref_quantize_q8_0(const float* x, uint64_t stride, void* y, int64_t k) {
  kq::quantize_row_q8_0_strided(x, stride, static_cast<kq::block_q8_0*>(y), k);
}
// weight quantizer the reference owns (src/emel/kernel/detail.hpp:699-…)
void ref_quantize_q4_0(const float* x, void* y, int64_t k) {
  kq::quantize_row_q4_0_ref(x, static_cast<kq::block_q4_0*>(y), k);
}

// ---- dequantizers (src/emel/kernel/detail.hpp:487-690)
int ref_dequantize_row(int type, const void* x, float* y, int64_t k) {
  switch (type) {
    case EMELB_Q4_0:
      kq::dequantize_row_q4_0(static_cast<const kq::block_q4_0*>(x), y, k);
      return 1;
    case EMELB_Q8_0:
      kq::dequantize_row_q8_0(static_cast<const kq::block_q8_0*>(x), y, k);
      return 1;
    case EMELB_Q4_K:
      kq::dequantize_row_q4_k(static_cast<const kq::block_q4_k*>(x), y, k);
      return 1;
    case EMELB_Q6_K:
      kq::dequantize_row_q6_k(static_cast<const kq::block_q6_k*>(x), y, k);
      return 1;
    default:
      return 0;
  }
}

// ---- guards (src/emel/kernel/detail.hpp:1919-1927, 3843-3872, 3573-3606,
//      4346-4390): validate_dispatch_request && can_run_*
int ref_can_run(uint32_t op_code, const emelb_op* op) {
  if (op_code == EMELB_OP_MUL_MAT) {
    const auto r = to_op<ev::op_mul_mat>(*op);
    return kd::validate_dispatch_request(r) && kd::can_run_mul_mat(r);
  }
  if (op_code == EMELB_OP_MUL_MAT_ARGMAX) {
    auto r = to_op<ev::op_mul_mat_argmax>(*op);
    r.index_out = op->index_out;
    return kd::validate_dispatch_request(r) && kd::can_run_mul_mat_argmax(r);
  }
  if (op_code == EMELB_OP_FLASH_ATTN_EXT) {
    const auto r = to_op<ev::op_flash_attn_ext>(*op);
    return kd::validate_dispatch_request(r) && kd::can_run_flash_attn_ext(r);
  }
  // the x86 actor's guard for these: validate_dispatch_request && can_run_backend_request
  // (src/emel/kernel/x86_64/guards.hpp valid_op; src/emel/kernel/detail.hpp:5315-5335)
  if (op_code == EMELB_OP_RMS_NORM) {
    const auto r = to_op<ev::op_rms_norm>(*op);
    return kd::validate_dispatch_request(r) && kd::can_run_backend_request(r);
  }
  if (op_code == EMELB_OP_ROPE) {
    const auto r = to_op<ev::op_rope>(*op);
    return kd::validate_dispatch_request(r) && kd::can_run_backend_request(r);
  }
  if (op_code == EMELB_OP_GLU) {
    const auto r = to_op<ev::op_glu>(*op);
    return kd::validate_dispatch_request(r) && kd::can_run_backend_request(r);
  }
  return 0;
}

// ---- op_rms_norm (src/emel/kernel/detail.hpp:4567-4602)
int ref_rms_norm(const emelb_op* op) {
  const auto r = to_op<ev::op_rms_norm>(*op);
  if (!(kd::validate_dispatch_request(r) && kd::can_run_norm_row_op(r))) return 0;
  return kd::run_rms_norm(r) ? 1 : 0;
}

// ---- op_rope, adjacent-pair (mode 0) and half-split (mode 2) variants (src/emel/kernel/detail.hpp:4706-4765)
int ref_rope(const emelb_op* op) {
  const auto r = to_op<ev::op_rope>(*op);
  if (!(kd::validate_dispatch_request(r) && kd::can_run_rope(r))) return 0;
  kd::rope_op_params p{};
  (void)kd::read_rope_params(r, p);
  if (p.mode == kd::rope_mode_norm) return kd::run_rope_as<false>(r) ? 1 : 0;
  if (p.mode == kd::rope_mode_neox) return kd::run_rope_as<true>(r) ? 1 : 0;
  return 0;
}

// ---- kernel::attention head-range event: the guard (src/emel/kernel/attention/guards.hpp:28-90) and the work
//      (src/emel/kernel/attention/actions.hpp:15-96) on the actor's own context type
namespace {
static emel::kernel::attention::event::head_range_request to_head_range(const emelb_head_range_request& r) {
  emel::kernel::attention::event::head_range_request q{};
  q.query = std::span<const float>(r.query, r.query_count);
  q.key_cache = std::span<const uint16_t>(r.key_cache, r.key_count);
  q.value_cache = std::span<const uint16_t>(r.value_cache, r.value_count);
  q.output = std::span<float>(r.output, r.output_count);
  q.layer_offset = r.layer_offset;
  q.hidden_dim = r.hidden_dim;
  q.head_dim = r.head_dim;
  q.head_begin = r.head_begin;
  q.head_end = r.head_end;
  q.position_capacity = r.position_capacity;
  q.physical_begin = r.physical_begin;
  q.valid_positions = r.valid_positions;
  return q;
}
}  // namespace

int ref_head_range_can_run(const emelb_head_range_request* r) {
  return emel::kernel::attention::guard::guard_request_shape_supported(to_head_range(*r)) ? 1 : 0;
}

int ref_head_range(const emelb_head_range_request* r) {
  namespace ka = emel::kernel::attention;
  const auto q = to_head_range(*r);
  if (!ka::guard::guard_request_shape_supported(q)) return 0;
  static thread_local ka::action::context ctx;
  ka::event::dispatch_result result{};
  ka::event::execute ev(q, result);
  ka::action::effect_execute_head_range{}(ev, ctx);
  return result.accepted ? 1 : 0;
}

// ---- op_mul_mat, scalar shared route (src/emel/kernel/detail.hpp:3356-3571)
int ref_mul_mat_scalar(const emelb_op* op) {
  const auto r = to_op<ev::op_mul_mat>(*op);
  if (!(kd::validate_dispatch_request(r) && kd::can_run_mul_mat(r))) return 0;
  return kd::run_mul_mat(r) ? 1 : 0;
}

// ---- op_mul_mat, AVX2/FMA route
//      (src/emel/kernel/x86_64/actions.hpp:1186-1326)
int ref_mul_mat_avx2(const emelb_op* op) {
  const auto r = to_op<ev::op_mul_mat>(*op);
  if (!(kd::validate_dispatch_request(r) && kd::can_run_mul_mat(r))) return 0;
  switch (op->src0.type) {
    case EMELB_Q4_K:
      kx::execute_avx2_fma_mul_mat_q4_k_q8_k_unchecked(r);
      return 1;
    case EMELB_Q6_K:
      kx::execute_avx2_fma_mul_mat_q6_k_q8_k_unchecked(r);
      return 1;
    case EMELB_Q8_0:
      kx::execute_avx2_fma_mul_mat_q8_0_q8_0_unchecked(r);
      return 1;
    case EMELB_Q4_0:
      kx::execute_avx2_fma_mul_mat_q4_0_q8_0_unchecked(r);
      return 1;
    default:
      return 0;
  }
}

// Row-sliced fork/join of the AVX2 route over std::thread: the reference's
// execute_parallel (src/emel/kernel/matmul/actions.hpp:48-67, 107-136;
// src/emel/kernel/matmul/detail.hpp:36-54) needs its un-vendored scheduler,
// so the slicing arithmetic is restated here and each lane runs the
// reference's own AVX2 driver on its slice.
int ref_mul_mat_avx2_lanes(const emelb_op* op, uint32_t lanes) {
  if (lanes <= 1) return ref_mul_mat_avx2(op);
  const uint64_t rows = op->src0.ne[1];
  std::vector<emelb_op> sliced;
  for (uint32_t lane = 0; lane < lanes; ++lane) {
    const uint64_t per = rows / lanes, extra = rows % lanes;
    const uint64_t begin = lane * per + (lane < extra ? lane : extra);
    const uint64_t count = per + (lane < extra ? 1u : 0u);
    if (count == 0) continue;
    emelb_op s = *op;
    s.src0.data = static_cast<const uint8_t*>(op->src0.data) + begin * op->src0.nb[1];
    s.src0.ne[1] = count;
    s.src0.nb[2] = op->src0.nb[1] * count;
    s.src0.nb[3] = s.src0.nb[2];
    s.dst.data = static_cast<const uint8_t*>(op->dst.data) + begin * op->dst.nb[1];
    s.dst.ne[1] = count;
    s.dst.nb[2] = op->dst.nb[1] * count;
    s.dst.nb[3] = s.dst.nb[2];
    sliced.push_back(s);
  }
  std::vector<int> ok(sliced.size(), 1);
  std::vector<std::thread> workers;
  for (size_t lane = 1; lane < sliced.size(); ++lane) {
    workers.emplace_back([&, lane] { ok[lane] = ref_mul_mat_avx2(&sliced[lane]); });
  }
  ok[0] = ref_mul_mat_avx2(&sliced[0]);
  for (auto& w : workers) w.join();
  for (int v : ok) {
    if (!v) return 0;
  }
  return 1;
}

// ---- op_mul_mat_argmax (src/emel/kernel/detail.hpp:3608-3731)
int ref_mul_mat_argmax(const emelb_op* op) {
  auto r = to_op<ev::op_mul_mat_argmax>(*op);
  r.index_out = op->index_out;
  if (!kd::validate_dispatch_request(r)) return 0;
  return kd::run_mul_mat_argmax(r) ? 1 : 0;
}

// ---- op_flash_attn_ext, scalar (src/emel/kernel/detail.hpp:5238-5300)
int ref_flash_attn_scalar(const emelb_op* op) {
  const auto r = to_op<ev::op_flash_attn_ext>(*op);
  if (!kd::validate_dispatch_request(r)) return 0;
  static thread_local kd::flash_attn_workspace ws{};
  return kd::run_flash_attn_ext_active_kv_with_workspace(r, ws) ? 1 : 0;
}

// ---- op_flash_attn_ext, AVX2/FMA/F16C one-chunk route
//      (src/emel/kernel/x86_64/actions.hpp:1575-1641)
int ref_flash_attn_avx2(const emelb_op* op) {
  const auto r = to_op<ev::op_flash_attn_ext>(*op);
  if (!kd::validate_dispatch_request(r)) return 0;
  static thread_local kd::flash_attn_workspace ws{};
  if (!kd::can_run_flash_attn_ext_with_workspace(r, ws)) return 0;
  kx::run_flash_attn_ext_f16kv_one_chunk_avx2_fma_f16c_unchecked(r, ws);
  return 1;
}

// ---- single-row dots, for SIMD==scalar checks
//      (tests/kernel/x86_64_tests.cpp:330-354, 536-654, 896-920)
float ref_row_dot_scalar(int type, const void* lhs, const void* rhs, uint64_t blocks) {
  switch (type) {
    case EMELB_Q4_K:
      return kd::dot_q4_k_q8_k_row_scalar(static_cast<const kq::block_q4_k*>(lhs),
                                          static_cast<const kq::block_q8_k*>(rhs), blocks);
    case EMELB_Q6_K:
      return kd::dot_q6_k_q8_k_row_scalar(static_cast<const kq::block_q6_k*>(lhs),
                                          static_cast<const kq::block_q8_k*>(rhs), blocks);
    case EMELB_Q8_0:
      return kd::dot_q8_0_q8_0_row_scalar(static_cast<const kq::block_q8_0*>(lhs),
                                          static_cast<const kq::block_q8_0*>(rhs), blocks);
    case EMELB_Q4_0:
      return kd::dot_q4_0_q8_0_row_scalar(static_cast<const kq::block_q4_0*>(lhs),
                                          static_cast<const kq::block_q8_0*>(rhs), blocks);
    default:
      return 0.0f;
  }
}

float ref_row_dot_avx2(int type, const void* lhs, const void* rhs, uint64_t blocks) {
  switch (type) {
    case EMELB_Q4_K:
      return kx::dot_q4_k_q8_k_row_avx2_fma(static_cast<const kq::block_q4_k*>(lhs),
                                            static_cast<const kq::block_q8_k*>(rhs), blocks);
    case EMELB_Q6_K:
      return kx::dot_q6_k_q8_k_row_avx2_fma(static_cast<const kq::block_q6_k*>(lhs),
                                            static_cast<const kq::block_q8_k*>(rhs), blocks);
    case EMELB_Q8_0:
      return kx::dot_q8_0_q8_0_row_avx2_fma(static_cast<const kq::block_q8_0*>(lhs),
                                            static_cast<const kq::block_q8_0*>(rhs), blocks);
    case EMELB_Q4_0:
      return kx::dot_q4_0_q8_0_row_avx2_fma(static_cast<const kq::block_q4_0*>(lhs),
                                            static_cast<const kq::block_q8_0*>(rhs), blocks);
    default:
      return 0.0f;
  }
}

int ref_host_has_avx2_fma_f16c(void) {
  return kx::detect_avx2() && kx::detect_fma() ? 1 : 0;
}

// ---- GGUF loader (src/emel/gguf/loader/detail.hpp:419-733).  The loader's state
// machine needs a header-only dependency that is not in the checkout, so the two
// functions it dispatches to are called directly, behind the request guard it
// applies first (an absent or empty image is invalid_request,
// src/emel/gguf/loader/guards.hpp:9-11, 33-43).
// req_out: {tensor_count, kv_count, max_key_bytes, max_value_bytes} then tensor_data_bytes
uint32_t ref_gguf_probe(const uint8_t* image, uint64_t bytes, uint32_t* req4_out, uint64_t* data_bytes_out) {
  namespace gl = ::emel::gguf::loader;
  if (image == nullptr || bytes == 0) return static_cast<uint32_t>(gl::error::invalid_request);
  gl::requirements req{};
  const auto err = gl::detail::probe_requirements(std::span<const uint8_t>{image, bytes}, req);
  req4_out[0] = req.tensor_count;
  req4_out[1] = req.kv_count;
  req4_out[2] = req.max_key_bytes;
  req4_out[3] = req.max_value_bytes;
  *data_bytes_out = req.tensor_data_bytes;
  return static_cast<uint32_t>(err);
}

// probe + bind + parse with exactly the storage the probe asked for.  Outputs, when
// the pointers are non-null and the parse succeeded:
//   kv_out[i*5..]     = {key_offset, key_length, value_offset, value_length, value_type}
//                       (offsets into arena_out, which must hold kv_count*(max_key+max_value) bytes)
//   tensor_out[i*11..] = {name_offset, name_length, type, n_dims, dims[4], data_offset, file_offset, data_size}
uint32_t ref_gguf_parse(const uint8_t* image, uint64_t bytes, uint8_t* arena_out, uint32_t* kv_out,
                        uint64_t* tensor_out) {
  namespace gl = ::emel::gguf::loader;
  if (image == nullptr || bytes == 0) return static_cast<uint32_t>(gl::error::invalid_request);
  const std::span<const uint8_t> file{image, bytes};
  gl::requirements req{};
  auto err = gl::detail::probe_requirements(file, req);
  if (err != 0) return static_cast<uint32_t>(err);
  std::vector<uint8_t> arena(gl::detail::required_kv_arena_bytes(req));
  std::vector<gl::kv_entry> kvs(req.kv_count);
  std::vector<::emel::model::data::tensor_record> tensors(req.tensor_count);
  err = gl::detail::parse_bound_storage(file, arena, kvs, tensors, req);
  if (err != 0) return static_cast<uint32_t>(err);
  if (arena_out != nullptr && !arena.empty()) std::memcpy(arena_out, arena.data(), arena.size());
  if (kv_out != nullptr) {
    for (size_t i = 0; i < kvs.size(); ++i) {
      const gl::kv_entry& e = kvs[i];
      const uint32_t row[5] = {e.key_offset, e.key_length, e.value_offset, e.value_length, e.value_type};
      std::memcpy(kv_out + i * 5, row, sizeof(row));
    }
  }
  if (tensor_out != nullptr) {
    for (size_t i = 0; i < tensors.size(); ++i) {
      const auto& t = tensors[i];
      uint64_t* row = tensor_out + i * 11;
      row[0] = t.name_offset;
      row[1] = t.name_length;
      row[2] = static_cast<uint64_t>(static_cast<int64_t>(t.type));
      row[3] = static_cast<uint64_t>(static_cast<int64_t>(t.n_dims));
      for (int d = 0; d < 4; ++d) row[4 + d] = static_cast<uint64_t>(t.dims[d]);
      row[8] = t.data_offset;
      row[9] = t.file_offset;
      row[10] = t.data_size;
      if (t.data != image + t.file_offset) return 0x8000u;  // the record must point into the image
    }
  }
  return 0u;
}

}  // extern "C"
