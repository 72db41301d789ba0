// Compile-and-run check of emel.cpp_b200/cuda_sm.hpp against the reference's own
// event headers: the adapter must accept the reference's op event types as they
// are.  Without a GPU the actor is not engaged and every dispatch is rejected.
#include <array>
#include <cstdio>

#include "../emel.cpp_b200/cuda_sm.hpp"

int main() {
  namespace ev = emel::kernel::event;
  emel::kernel::cuda::sm machine{0};
  std::array<float, 256> x{};
  std::array<unsigned char, 144> w{};
  float y = 0.0f;
  ev::op_mul_mat mm{};
  mm.src0.data = w.data();
  mm.src0.type = ev::dtype::q4_k;
  mm.src0.ne = {256, 1, 1, 1};
  mm.src0.nb = {1, 144, 144, 144};
  mm.src1.data = x.data();
  mm.src1.type = ev::dtype::f32;
  mm.src1.ne = {1, 256, 1, 1};
  mm.src1.nb = {4, 4, 1024, 1024};
  mm.dst.data = &y;
  mm.dst.type = ev::dtype::f32;
  mm.dst.ne = {1, 1, 1, 1};
  mm.dst.nb = {4, 4, 4, 4};
  const bool accepted = machine.process_event(mm);
  // the other attention actor's event type is accepted as it is too (rejected here: no device)
  emel::kernel::attention::event::head_range_request hr{};
  emel::kernel::attention::event::dispatch_result hr_result{};
  emel::kernel::attention::event::execute hr_event(hr, hr_result);
  const bool hr_accepted = machine.process_event(hr_event);
  if (hr_accepted || hr_result.accepted) return 1;
  ev::op_add other{};
  const bool other_accepted = machine.process_event(other);
  std::printf("engaged=%d accepted=%d error=%u other=%d other_error=%u\n", machine.engaged() ? 1 : 0, accepted ? 1 : 0,
              static_cast<unsigned>(machine.last_error()), other_accepted ? 1 : 0,
              static_cast<unsigned>(emel::kernel::error::unsupported_op));
  return 0;
}
