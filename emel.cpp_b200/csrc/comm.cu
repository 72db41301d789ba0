// Exchange step of the row-sharded path.  The reference forks one op_mul_mat into
// disjoint destination-row intervals that share the right-hand side and joins
// them in memory (src/emel/kernel/matmul/detail.hpp:36-57,
// src/emel/kernel/matmul/actions.hpp:48-67).  With one process per GPU the join
// is an all-gather of each rank's f32 row interval: every element is computed by
// exactly one rank with the arithmetic of the unsharded kernel, so the gathered
// vector is the unsharded result bit for bit.  NCCL over NVLink carries it; the
// call is stream-ordered and may be captured into the per-token graph.
#include <cstring>

#include "../../include/emelb.h"
#include "ctx.h"

#if defined(EMELB_HAVE_NCCL)
#include <nccl.h>
#endif

using namespace emelb;

namespace emelb {

cudaError_t comm_all_gather_bytes(emelb_ctx* c, void* buf, size_t bytes_per_rank, cudaStream_t st) {
#if defined(EMELB_HAVE_NCCL)
  if (!c->comm || c->comm_world <= 1) return cudaSuccess;
  char* base = static_cast<char*>(buf);
  const ncclResult_t r = ncclAllGather(base + (size_t)c->comm_rank * bytes_per_rank, base, bytes_per_rank, ncclChar,
                                       static_cast<ncclComm_t>(c->comm), st);
  return r == ncclSuccess ? cudaSuccess : cudaErrorUnknown;
#else
  (void)c; (void)buf; (void)bytes_per_rank; (void)st;
  return cudaErrorNotSupported;
#endif
}

// ---- peer-store join (same node): each rank copies its row interval straight into every peer's copy of the
// vector over NVLink, raises a per-sender sequence flag on the peer, and waits for every peer's flag.  One small
// kernel per join instead of a collective launch; plain peer stores and loads (no multimem), so a rank that
// leaves between steps cannot fault its peers.  Waits are bounded: on a timeout the status word is raised and
// the kernel returns.
namespace {

constexpr int kPeerWaitSpins = 1 << 30;   // the wall-clock limit (PeerGatherArgs::wait_ns) is the effective bound

__global__ void __launch_bounds__(1024) peer_gather_kernel(PeerGatherArgs a) {
  const int peers = a.world - 1;
  // 1. my interval -> every peer's buffer (16-byte stores; intervals are multiples of 16 bytes)
  const uint4* src = reinterpret_cast<const uint4*>(a.local_base + a.offset_bytes);
  const size_t n16 = a.bytes_per_rank / 16;
  for (size_t i = threadIdx.x; i < n16 * (size_t)peers; i += blockDim.x) {
    const int pi = (int)(i / n16);
    const size_t j = i - (size_t)pi * n16;
    const int peer = pi < a.rank ? pi : pi + 1;
    reinterpret_cast<uint4*>(a.peer_base[peer] + a.offset_bytes)[j] = src[j];
  }
  __threadfence_system();
  __syncthreads();
  // 2. advance my sequence number and publish it on every peer
  __shared__ unsigned int s_seq;
  if (threadIdx.x == 0) s_seq = ++(*a.seq);
  __syncthreads();
  const unsigned int seq = s_seq;
  if (threadIdx.x < a.world && (int)threadIdx.x != a.rank) {
    unsigned int* flag = reinterpret_cast<unsigned int*>(a.peer_base[threadIdx.x] + a.flags_offset) + a.rank;
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(flag), "r"(seq) : "memory");
  }
  // 3. wait until every peer's data for this join has landed here
  if (threadIdx.x < a.world && (int)threadIdx.x != a.rank) {
    const unsigned int* flag = reinterpret_cast<const unsigned int*>(a.local_base + a.flags_offset) + threadIdx.x;
    unsigned long long t0 = 0;
    bool ok = false;
    for (int spins = 0; spins < kPeerWaitSpins; ++spins) {
      unsigned int v;
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
      if ((int)(v - seq) >= 0) { ok = true; break; }
      if ((spins & 1023) == 1023) {
        if (a.status && *reinterpret_cast<volatile int*>(a.status) != 0) break;   // an earlier wait already ran out
        unsigned long long now;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
        if (t0 == 0) t0 = now;
        else if (now - t0 > a.wait_ns) break;
      }
    }
    if (!ok && a.status) atomicExch(a.status, 1);
  }
}

}  // namespace

cudaError_t launch_peer_gather(const PeerGatherArgs& a, cudaStream_t st) {
  peer_gather_kernel<<<1, 1024, 0, st>>>(a);
  return cudaGetLastError();
}

void comm_release(emelb_ctx* c) {
#if defined(EMELB_HAVE_NCCL)
  if (c->comm) ncclCommDestroy(static_cast<ncclComm_t>(c->comm));
#endif
  c->comm = nullptr;
  c->comm_world = 1;
  c->comm_rank = 0;
}

}  // namespace emelb

extern "C" {

uint32_t emelb_comm_unique_id(uint8_t* id_out, uint64_t id_bytes) {
#if defined(EMELB_HAVE_NCCL)
  if (!id_out || id_bytes < EMELB_COMM_ID_BYTES) return EMELB_INVALID_REQUEST;
  static_assert(sizeof(ncclUniqueId) <= EMELB_COMM_ID_BYTES, "id buffer too small");
  ncclUniqueId id;
  if (ncclGetUniqueId(&id) != ncclSuccess) return EMELB_INTERNAL_ERROR;
  std::memset(id_out, 0, EMELB_COMM_ID_BYTES);
  std::memcpy(id_out, &id, sizeof id);
  return EMELB_OK;
#else
  (void)id_out; (void)id_bytes;
  return EMELB_UNSUPPORTED_OP;
#endif
}

uint32_t emelb_comm_init(emelb_ctx* c, int32_t rank, int32_t world, const uint8_t* id, uint64_t id_bytes) {
#if defined(EMELB_HAVE_NCCL)
  if (!c || !id || id_bytes < EMELB_COMM_ID_BYTES || world < 1 || rank < 0 || rank >= world || c->comm) return EMELB_INVALID_REQUEST;
  cudaSetDevice(c->device);
  ncclUniqueId uid;
  std::memcpy(&uid, id, sizeof uid);
  ncclComm_t comm = nullptr;
  if (ncclCommInitRank(&comm, world, uid, rank) != ncclSuccess) return EMELB_INTERNAL_ERROR;
  c->comm = comm;
  c->comm_rank = rank;
  c->comm_world = world;
  return EMELB_OK;
#else
  (void)c; (void)rank; (void)world; (void)id; (void)id_bytes;
  return EMELB_UNSUPPORTED_OP;
#endif
}

uint32_t emelb_set_peer_wait_ms(emelb_ctx* c, uint32_t limit_ms) {
  if (!c || limit_ms == 0) return EMELB_INVALID_REQUEST;
  c->peer_wait_ns = (unsigned long long)limit_ms * 1000000ull;
  return EMELB_OK;
}

uint32_t emelb_selftest_wait_timeout(emelb_ctx* c, uint32_t limit_ms) {
  if (!c || limit_ms == 0 || limit_ms > 10000 || c->stage_in_bytes < 8192) return EMELB_INVALID_REQUEST;
  cudaSetDevice(c->device);
  // a join of two "ranks" that are both this context's own staging buffer: rank 0 publishes its flag and waits
  // for rank 1's, which nobody raises
  char* arena = static_cast<char*>(c->stage_in);
  if (cudaMemsetAsync(arena, 0, 8192, c->stream) != cudaSuccess) return EMELB_INTERNAL_ERROR;
  PeerGatherArgs a{};
  a.local_base = arena;
  a.peer_base[0] = arena;
  a.peer_base[1] = arena;
  a.offset_bytes = 4096;
  a.bytes_per_rank = 256;
  a.flags_offset = 0;
  a.seq = reinterpret_cast<unsigned int*>(arena + 1024);
  a.rank = 0;
  a.world = 2;
  a.status = c->status_word();
  a.wait_ns = (unsigned long long)limit_ms * 1000000ull;
  const cudaError_t e = launch_peer_gather(a, c->stream);
  c->diag.kernel_launches += 1;
  if (e != cudaSuccess) {
    c->last_cuda_error = (int)e;
    return EMELB_INTERNAL_ERROR;
  }
  return EMELB_OK;
}

uint32_t emelb_comm_destroy(emelb_ctx* c) {
  if (!c) return EMELB_INVALID_REQUEST;
  cudaSetDevice(c->device);
  if (c->stream) cudaStreamSynchronize(c->stream);
  comm_release(c);
  return EMELB_OK;
}

uint32_t emelb_all_gather_rows(emelb_ctx* c, float* dst_dev, uint64_t rows_per_rank, uint64_t row_floats) {
  if (!c || !dst_dev || rows_per_rank == 0 || row_floats == 0) return EMELB_INVALID_REQUEST;
  if (!c->comm) return c->comm_world <= 1 ? EMELB_OK : EMELB_INVALID_REQUEST;
  cudaSetDevice(c->device);
  const cudaError_t e = comm_all_gather_bytes(c, dst_dev, (size_t)(rows_per_rank * row_floats) * sizeof(float), c->stream);
  if (e != cudaSuccess) {
    c->last_cuda_error = (int)e;
    return EMELB_INTERNAL_ERROR;
  }
  return EMELB_OK;
}

}  // extern "C"
