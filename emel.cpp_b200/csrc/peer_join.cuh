// Device side of the joins by peer stores (JoinOut / JoinIn in kernels.h).
#pragma once

#include "kernels.h"

namespace emelb {

// One warp: the Q8_K block it has just quantized (q8_k_block_warp's outputs) goes into every rank's planes of the
// joined vector, at 256-block `blk` of that vector.
__device__ __forceinline__ void join_store_q8_k_block(const JoinOut& j, int blk, int lane, uint32_t lo, uint32_t hi, int bsum16,
                                                      float d) {
#pragma unroll
  for (int g = 0; g < kMaxPeers; ++g) {
    if (g < j.world) {
      char* base = j.base[g];
      *reinterpret_cast<uint2*>(base + j.qs_offset + (int64_t)blk * 256 + 8 * lane) = make_uint2(lo, hi);
      if ((lane & 1) == 0) reinterpret_cast<int16_t*>(base + j.bsums_offset)[blk * 16 + (lane >> 1)] = (int16_t)bsum16;
      if (lane == 0) reinterpret_cast<float*>(base + j.d_offset)[blk] = d;
    }
  }
}

// One thread, after every block's stores to the peers are fenced and counted: advance this rank's sequence
// number of the join and publish it on every peer.
__device__ __forceinline__ void join_raise(const JoinOut& j) {
  __threadfence_system();
  const unsigned seq = ++(*j.seq);
#pragma unroll
  for (int g = 0; g < kMaxPeers; ++g) {
    if (g < j.world && g != j.rank) {
      unsigned* flag = reinterpret_cast<unsigned*>(j.base[g] + j.flag_offset) + j.rank;
      asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(flag), "r"(seq) : "memory");
    }
  }
}

// Every thread of the CTA, at the end of a kernel whose blocks stored to the peers and that has no block counter
// of its own: the last block to arrive raises the flag.
__device__ __forceinline__ void join_publish(const JoinOut& j, unsigned nblocks) {
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    if (atomicAdd(j.done, 1) == (int)nblocks - 1) {
      *j.done = 0;
      join_raise(j);
    }
  }
}

// Every thread of the CTA, before the first read of the joined vector: threads 0 .. world-1 each watch one
// peer's flag.  The wait is bounded by wall-clock time; when it runs out the status word is raised and the
// kernel carries on (with whatever the vector holds), so the stream drains and the host reads the failure.
__device__ __forceinline__ void join_wait(const JoinIn& j, int* status) {
  if ((int)threadIdx.x < j.world && (int)threadIdx.x != j.rank) {
    const unsigned want = *reinterpret_cast<const volatile unsigned*>(j.seq);
    const unsigned* flag = j.flags + threadIdx.x;
    unsigned long long t0 = 0;
    bool ok = false;
    for (int spins = 0; spins < (1 << 30); ++spins) {
      unsigned v;
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
      if ((int)(v - want) >= 0) { ok = true; break; }
      __nanosleep(100);   // every CTA of the launch watches the same words: leave the line to the incoming store
      if ((spins & 255) == 255) {
        // a wait that already ran out anywhere on this context ends every later one at once: the step is lost
        // anyway, and the stream must drain in bounded time
        if (status && *reinterpret_cast<volatile int*>(status) != 0) break;
        unsigned long long now;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
        if (t0 == 0) t0 = now;
        else if (now - t0 > j.wait_ns) break;
      }
    }
    if (!ok && status) atomicExch(status, 1);
  }
  __syncthreads();
}

}  // namespace emelb
