// emel::kernel::cuda::sm — the host-side mirror of the reference's kernel actor
// for the B200 backend.  It exposes the overload set a backend in
// kernel::any's sm_list must have, `bool process_event(const event::op_X&)`
// (src/emel/kernel/x86_64/sm.hpp:1198-1211; src/emel/kernel/any.hpp:76-80), for
// the three ops on the quantized matrix-product path and forwards each to the
// C-ABI of include/emelb.h.  Everything else is rejected with unsupported_op,
// the way a backend without a matching transition row rejects an event.
//
// Compiles against the reference's own event headers (events.hpp needs none of
// the state-machine library):
//   g++ -std=c++20 -I<reference>/src -I<reference>/include -I<this repo>/include \
//       -fsyntax-only emel.cpp_b200/cuda_sm.hpp
// In the reference tree the same class would be wrapped as an `emel::sm<model,
// context>` whose single `ready` state has one guard/action row per op.
#pragma once

#include <cstdint>
#include <cstring>

#include "emel/kernel/attention/events.hpp"
#include "emel/kernel/errors.hpp"
#include "emel/kernel/events.hpp"

#include "emelb.h"

namespace emel::kernel::cuda {

namespace detail {

inline emelb_view to_view(const ::emel::kernel::event::tensor_view& v) noexcept {
  emelb_view out{};
  out.data = v.data;
  out.type = static_cast<uint8_t>(v.type);
  for (int i = 0; i < 4; ++i) {
    out.ne[i] = v.ne[static_cast<size_t>(i)];
    out.nb[i] = v.nb[static_cast<size_t>(i)];
  }
  return out;
}

inline emelb_view to_view(const ::emel::kernel::event::tensor_view_mut& v) noexcept {
  emelb_view out{};
  out.data = v.data;
  out.type = static_cast<uint8_t>(v.type);
  for (int i = 0; i < 4; ++i) {
    out.ne[i] = v.ne[static_cast<size_t>(i)];
    out.nb[i] = v.nb[static_cast<size_t>(i)];
  }
  return out;
}

template <class op_type>
inline emelb_op to_op(const op_type& ev) noexcept {
  emelb_op out{};
  out.src0 = to_view(ev.src0);
  out.src1 = to_view(ev.src1);
  out.src2 = to_view(ev.src2);
  out.dst = to_view(ev.dst);
  std::memcpy(out.op_params, ev.op_params.data(), sizeof(out.op_params));
  out.op_params_size = ev.op_params_size;
  out.index_out = nullptr;
  return out;
}

}  // namespace detail

class sm {
 public:
  // one actor = one backend context on `device`; engaged() is false when the
  // context could not be created (no device, out of memory)
  explicit sm(const int device = 0) noexcept { last_error_ = emelb_create(device, &ctx_); }
  sm(const sm&) = delete;
  sm& operator=(const sm&) = delete;
  ~sm() {
    if (ctx_ != nullptr) {
      emelb_destroy(ctx_);
    }
  }

  bool engaged() const noexcept { return ctx_ != nullptr; }
  emelb_ctx* context() noexcept { return ctx_; }

  // accepted <=> error == none (src/emel/kernel/x86_64/sm.hpp:1327-1331)
  bool process_event(const ::emel::kernel::event::op_mul_mat& ev) noexcept {
    const emelb_op op = detail::to_op(ev);
    return finish(emelb_mul_mat(ctx_, &op));
  }

  bool process_event(const ::emel::kernel::event::op_mul_mat_argmax& ev) noexcept {
    emelb_op op = detail::to_op(ev);
    op.index_out = ev.index_out;
    return finish(emelb_mul_mat_argmax(ctx_, &op));
  }

  bool process_event(const ::emel::kernel::event::op_flash_attn_ext& ev) noexcept {
    const emelb_op op = detail::to_op(ev);
    return finish(emelb_flash_attn_ext(ctx_, &op));
  }

  bool process_event(const ::emel::kernel::event::op_rms_norm& ev) noexcept {
    const emelb_op op = detail::to_op(ev);
    return finish(emelb_rms_norm(ctx_, &op));
  }

  bool process_event(const ::emel::kernel::event::op_rope& ev) noexcept {
    const emelb_op op = detail::to_op(ev);
    return finish(emelb_rope(ctx_, &op));
  }

  // rejected as by the reference's own backends (no row executes op_glu there)
  bool process_event(const ::emel::kernel::event::op_glu& ev) noexcept {
    const emelb_op op = detail::to_op(ev);
    return finish(emelb_glu(ctx_, &op));
  }

  // kernel::attention's head-range event (src/emel/kernel/attention/events.hpp:33-43): the result's `accepted`
  // is what effect_execute_head_range / effect_reject_execute leave there
  bool process_event(const ::emel::kernel::attention::event::execute& ev) noexcept {
    const auto& r = ev.request;
    emelb_head_range_request q{};
    q.query = r.query.data();
    q.query_count = r.query.size();
    q.key_cache = r.key_cache.data();
    q.key_count = r.key_cache.size();
    q.value_cache = r.value_cache.data();
    q.value_count = r.value_cache.size();
    q.output = r.output.data();
    q.output_count = r.output.size();
    q.layer_offset = r.layer_offset;
    q.hidden_dim = r.hidden_dim;
    q.head_dim = r.head_dim;
    q.head_begin = r.head_begin;
    q.head_end = r.head_end;
    q.position_capacity = r.position_capacity;
    q.physical_begin = r.physical_begin;
    q.valid_positions = r.valid_positions;
    ev.result.accepted = finish(emelb_attention_head_range(ctx_, &q));
    return ev.result.accepted;
  }

  // every other op event: no row in this backend
  template <class event_type>
  bool process_event(const event_type&) noexcept {
    return finish(EMELB_UNSUPPORTED_OP);
  }

  // event::capture_diagnostics (src/emel/kernel/any.hpp:38-74)
  bool process_event(const ::emel::kernel::event::capture_diagnostics& ev) noexcept {
    emelb_diag d{};
    if (emelb_diagnostics(ctx_, &d) != EMELB_OK) {
      return false;
    }
    ev.out.optimized_flash_dispatch_calls = d.optimized_flash_dispatch_calls;
    ev.out.shared_flash_dispatch_calls = d.shared_flash_dispatch_calls;
    ev.out.optimized_q4_dispatch_calls = d.optimized_q4_dispatch_calls;
    ev.out.optimized_q4_vector_dispatch_calls = d.optimized_q4_vector_dispatch_calls;
    ev.out.optimized_q6_dispatch_calls = d.optimized_q6_dispatch_calls;
    ev.out.optimized_q6_vector_dispatch_calls = d.optimized_q6_vector_dispatch_calls;
    ev.out.optimized_q6_vector_argmax_dispatch_calls = d.optimized_q6_vector_argmax_dispatch_calls;
    return true;
  }

  ::emel::kernel::error last_error() const noexcept {
    return static_cast<::emel::kernel::error>(last_error_);
  }

  // residency seam: io::loader strategy `external_buffer`
  // (src/emel/io/loader/events.hpp:25-31) -> the span is mirrored in HBM and
  // later views may keep carrying the host address
  bool bind_external_buffer(const int32_t tensor_id, const void* host, const uint64_t bytes,
                            const int32_t tensor_type) noexcept {
    return finish(emelb_residency_upload(ctx_, tensor_id, host, bytes, tensor_type, nullptr));
  }
  bool evict(const int32_t tensor_id) noexcept { return finish(emelb_residency_evict(ctx_, tensor_id)); }

 private:
  bool finish(const uint32_t err) noexcept {
    last_error_ = err;
    return err == EMELB_OK;
  }

  emelb_ctx* ctx_ = nullptr;
  uint32_t last_error_ = EMELB_OK;
};

}  // namespace emel::kernel::cuda
