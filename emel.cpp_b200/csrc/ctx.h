// The backend context behind include/emelb.h's opaque emelb_ctx: stream,
// persistent workspace, residency table and dispatch counters.  Its role is the
// one of a kernel actor's context in the reference
// (src/emel/kernel/x86_64/context.hpp:214-243): everything a dispatch needs is
// allocated once, up front.
#pragma once

#include <map>
#include <set>
#include <vector>

#include "../../include/emelb.h"
#include "kernels.h"

namespace emelb {

constexpr uint64_t kFlashPartFloats = 4u << 20;   // split-KV partial accumulators
constexpr uint64_t kFlashScoreFloats = 8u << 20;  // reference-order score rows

struct Resident {
  int state = EMELB_LIFECYCLE_UNBOUND;
  void* dev = nullptr;
  uint64_t bytes = 0;
  const void* host = nullptr;
  int32_t type = 0;
};

// one uploader thread's share of the page-locked staging ring (upload.cu)
struct UploadLane {
  cudaStream_t stream = nullptr;
  void* pinned[2] = {nullptr, nullptr};
  cudaEvent_t drained[2] = {nullptr, nullptr};
};

ActPlanes planes_view(const ActPlanesMut& m, int type, int K);
cudaError_t quantize_into_planes(int wtype, const float* x, int n, int ncols, int K, ActPlanesMut out, cudaStream_t st);

}  // namespace emelb

struct emelb_ctx;
namespace emelb {
// one span of a residency upload: `host` is the key and, when no file is named, the source
struct UploadSpan {
  int32_t tensor_id;
  const void* host;
  uint64_t bytes;
  int32_t tensor_type;
  uint64_t file_offset;  // of the span in the file `fd` names (unused when fd < 0)
  void* dev;             // filled by residency_upload_many
};
// spans -> their device buffers, complete on return.  Spans outside page-locked memory go through the
// staging ring in one pipeline over all of them; fd >= 0 names the file the spans map (read by pread).
cudaError_t upload_spans(emelb_ctx* c, const UploadSpan* spans, size_t count, int fd);
void upload_ring_release(emelb_ctx* c);
// emelb_residency_upload for several tensors at once: all or nothing
uint32_t residency_upload_many(emelb_ctx* c, UploadSpan* spans, size_t count, int fd);
}  // namespace emelb

struct emelb_ctx {
  int device = 0;
  int sm_count = 0;
  cudaStream_t stream = nullptr;
  int attention_mode = 0;
  int last_cuda_error = 0;
  // device staging for host-resident activations / results
  void* stage_in = nullptr;
  uint64_t stage_in_bytes = 0;
  void* stage_out = nullptr;
  uint64_t stage_out_bytes = 0;
  // quantized activation planes (scratch of op_mul_mat)
  int8_t* act_qs = nullptr;
  float* act_d = nullptr;
  int16_t* act_bsums = nullptr;
  uint64_t act_capacity = 0;  // elements
  uint8_t* tc_ws = nullptr;   // the many-column kernel's copy of the planes in operand order
  uint64_t tc_ws_bytes = 0;
  // shape of the activations emelb_prepare_rhs left in the planes (0 = none)
  uint64_t prepared_n = 0;
  uint64_t prepared_k = 0;
  bool prepared_k_family = false;
  // task counters of the streaming mat-vec kernel: kSchedSlots {next task, finished blocks} pairs used
  // in rotation (consecutive launches may overlap), then the status word (a bounded wait ran out)
  int* gemv_sched = nullptr;
  int sched_next = 0;
  int pdl = 0;  // launch decode-chain kernels with programmatic stream serialization
  int* next_sched() { int* p = gemv_sched + 2 * sched_next; sched_next = (sched_next + 1) % emelb::kSchedSlots; return p; }
  int* status_word() { return gemv_sched + 2 * emelb::kSchedSlots; }
  // scratch of the whole-token decode kernel's products: block values per row (rows whose K spans several
  // chunk pairs are completed through it) and row-group arrival counters, zero between launches
  float* bv_table = nullptr;
  uint64_t bv_table_floats = 0;
  int* grp_cnt = nullptr;
  uint64_t grp_cnt_ints = 0;
  // whole-token decode kernel: grid barrier {arrivals, generation, abort, -} and the attention units' arrival
  // counters (kTokenCounters ints), all zero between launches
  unsigned* token_bar = nullptr;
  int* token_cnt = nullptr;
  static constexpr int kTokenCounters = 1024;
  // argmax candidates and result cells
  float* part_val = nullptr;
  int* part_idx = nullptr;
  float* best_val = nullptr;
  int* best_idx = nullptr;
  // attention workspace
  float* fa_part_acc = nullptr;
  float* fa_part_ml = nullptr;
  float* fa_scores = nullptr;
  // residency: tensor id -> device copy; host span start -> tensor id
  std::map<int32_t, emelb::Resident> residents;
  std::map<uintptr_t, int32_t> by_host;
  std::set<void*> owned;
  std::map<uintptr_t, uint64_t> dev_ranges;  // device spans this context allocated (start -> bytes)
  bool capturing = false;
  std::vector<emelb::UploadLane> upload_lanes;  // created by the first large residency upload
  int upload_route = 0;    // EMELB_UPLOAD_RING / _PLAIN / _REGISTER (emelb_set_upload_route)
  int upload_threads = 0;  // 0: one per host core, at most 16
  // row-shard exchange (comm.cu): one communicator per context, one rank per GPU
  void* comm = nullptr;  // ncclComm_t
  int comm_rank = 0;
  int comm_world = 1;
  unsigned long long peer_wait_ns = emelb::kPeerWaitNsDefault;  // bound of a peer-store join's wait (emelb_set_peer_wait_ms)
  emelb_diag diag = {};
};
