// CPU harness for tests/test_expf_exact.py: compares emelb::expf_exact (the same
// source the CUDA kernels compile) with the host C library's expf over a strided
// sweep of all float bit patterns.  Prints the number of mismatches.
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <thread>
#include <vector>

#include "../emel.cpp_b200/csrc/expf_exact.h"

int main(int argc, char** argv) {
  const uint64_t stride = argc > 1 ? strtoull(argv[1], nullptr, 10) : 1;
  const unsigned nt = std::thread::hardware_concurrency() ? std::thread::hardware_concurrency() : 4;
  std::vector<uint64_t> bad(nt, 0), first(nt, 0);
  std::vector<std::thread> th;
  for (unsigned t = 0; t < nt; ++t) {
    th.emplace_back([&, t] {
      for (uint64_t u = t * stride; u < (1ull << 32); u += nt * stride) {
        const uint32_t bits = (uint32_t)u;
        float x;
        memcpy(&x, &bits, 4);
        const float a = expf(x), b = emelb::expf_exact(x);
        uint32_t ua, ub;
        memcpy(&ua, &a, 4);
        memcpy(&ub, &b, 4);
        const bool same = ua == ub || (a != a && b != b);
        if (!same) {
          if (!bad[t]) first[t] = u;
          ++bad[t];
        }
      }
    });
  }
  for (auto& x : th) x.join();
  uint64_t total = 0;
  for (unsigned t = 0; t < nt; ++t) {
    total += bad[t];
    if (bad[t]) fprintf(stderr, "first mismatch at bits %08llx\n", (unsigned long long)first[t]);
  }
  printf("%llu\n", (unsigned long long)total);
  return 0;
}
