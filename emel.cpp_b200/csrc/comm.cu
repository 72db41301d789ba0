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
