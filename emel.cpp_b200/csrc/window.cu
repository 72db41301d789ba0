// The layer streaming window with device slots (include/emelb_window.h).
//
// The plan arithmetic, the order of the bind decisions and the ring rules restate the reference's
// model::tensor::window (src/emel/model/tensor/window/detail.hpp:128-183, guards.hpp:13-186 and 296-470,
// actions.hpp:218-227 and 394-406).  A slot load is a device matter:
//   * source page-locked (tried at bind): a load is one asynchronous copy per extent on the window's own stream.
//     The copy waits for the event that marks the end of the slot's previous readers on the compute stream, and the
//     compute stream waits for the event behind the copy: the host thread never blocks;
//   * otherwise one I/O thread stages each extent in chunks through two page-locked buffers; an acquire of a layer that
//     is still loading waits for the thread on the host.
// Nothing here allocates in acquire.
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <condition_variable>
#include <cstring>
#include <deque>
#include <mutex>
#include <new>
#include <thread>
#include <vector>

#include "../../include/emelb_window.h"
#include "ctx.h"
#include "window.h"

namespace {

constexpr uint64_t kMaxMappingBytes = 1ull << 40;   // the reference's io::mmap cap on one mapping

enum Lifecycle { VACANT = 0, LOADING = 1, RESIDENT = 2, FAILED = 3 };   // detail.hpp:47-52

struct Slot {
  uint8_t* storage = nullptr;
  int layer = -1;
  int lifecycle = VACANT;
  cudaEvent_t loaded = nullptr;    // recorded on the copy stream behind the slot's last load
  cudaEvent_t released = nullptr;  // recorded on the compute stream when the slot's view was given up
};

uint64_t aligned(uint64_t bytes) { return (bytes + (EMELB_WINDOW_SLOT_ALIGNMENT - 1)) & ~uint64_t(EMELB_WINDOW_SLOT_ALIGNMENT - 1); }

}  // namespace

struct emelb_window {
  emelb_ctx* c = nullptr;
  bool bound = false, streaming = false;
  std::vector<emelb_window_layer> plan;
  Slot slots[EMELB_WINDOW_MAX_SLOTS];
  uint32_t slot_count = 0;
  uint64_t slot_capacity = 0;
  const uint8_t* source = nullptr;
  uint64_t source_bytes = 0;
  bool mapped_here = false;      // the window mapped the file itself
  bool page_locked = false;      // the copy engines can read the source in place
  void* locked_base = nullptr;   // start of the range this window page-locked itself (null: none)
  bool staged_only = false;
  uint32_t prefetch_depth = 0;
  uint64_t chunk = EMELB_WINDOW_DEFAULT_CHUNK_BYTES;
  int published_slot = -1;
  cudaStream_t copy_stream = nullptr;
  int fail_next = 0;
  emelb_window_stats stats{};
  // the staged route's I/O thread
  std::thread worker;
  std::mutex m;
  std::condition_variable cv;
  std::deque<int> jobs;          // slots to load, in submission order (slot.layer names the layer)
  bool busy = false, stop = false;
  void* pinned[2] = {nullptr, nullptr};
  cudaEvent_t drained[2] = {nullptr, nullptr};
};

namespace {

// detail.hpp:128-167: extents packed per layer at 64-byte aligned offsets; the slot capacity is the largest layer
void scan_layers(emelb_window* w, const emelb_window_request& r) {
  w->plan.assign(size_t(r.layer_count), emelb_window_layer{});
  uint64_t cursor = 0, widest = 0;
  for (uint64_t l = 0; l < r.layer_count; ++l) {
    emelb_window_layer& d = w->plan[size_t(l)];
    d.weight_count = r.layer_weight_counts[l];
    uint64_t at = 0, lo = ~0ull, hi = 0;
    for (uint32_t i = 0; i < d.weight_count; ++i) {
      emelb_window_extent e = r.extents[cursor++];
      e.slot_offset = at;
      at += aligned(e.byte_size);
      lo = e.file_offset < lo ? e.file_offset : lo;
      hi = e.file_offset + e.byte_size > hi ? e.file_offset + e.byte_size : hi;
      d.weights[i] = e;
    }
    d.slot_bytes = at;
    d.file_begin = d.weight_count ? lo : 0;
    d.file_span = d.weight_count ? hi - d.file_begin : 0;
    widest = at > widest ? at : widest;
  }
  w->slot_capacity = widest;
}

// guards.hpp:13-60
bool request_valid(const emelb_window_request& r) {
  const bool has_source = r.source != nullptr || (r.file_path != nullptr && r.file_path[0] != '\0');
  if (!has_source || r.file_size_bytes == 0) return false;
  if (r.layer_count == 0 || r.layer_count > EMELB_WINDOW_MAX_LAYERS) return false;
  if (!r.layer_weight_counts || !r.extents) return false;
  uint64_t total = 0;
  for (uint64_t l = 0; l < r.layer_count; ++l) {
    const uint16_t n = r.layer_weight_counts[l];
    if (n == 0 || n > EMELB_WINDOW_MAX_WEIGHTS_PER_LAYER) return false;
    total += n;
  }
  if (total != r.extent_count) return false;
  for (uint64_t i = 0; i < r.extent_count; ++i) {
    const emelb_window_extent& e = r.extents[i];
    if (e.byte_size == 0 || e.byte_size > r.file_size_bytes || e.file_offset > r.file_size_bytes - e.byte_size) return false;
  }
  return r.stage_chunk_bytes >= EMELB_WINDOW_MIN_CHUNK_BYTES && r.stage_chunk_bytes <= EMELB_WINDOW_MAX_CHUNK_BYTES;
}

bool map_source(emelb_window* w, const emelb_window_request& r) {
  if (r.file_size_bytes > kMaxMappingBytes) return false;
  if (r.source) {
    w->source = static_cast<const uint8_t*>(r.source);
    w->source_bytes = r.file_size_bytes;
    w->mapped_here = false;
    return true;
  }
  const int fd = ::open(r.file_path, O_RDONLY | O_CLOEXEC);
  if (fd < 0) return false;
  struct stat st{};
  void* p = MAP_FAILED;
  if (::fstat(fd, &st) == 0 && uint64_t(st.st_size) >= r.file_size_bytes)
    p = ::mmap(nullptr, size_t(r.file_size_bytes), PROT_READ, MAP_PRIVATE, fd, 0);
  ::close(fd);
  if (p == MAP_FAILED) return false;
  w->source = static_cast<const uint8_t*>(p);
  w->source_bytes = r.file_size_bytes;
  w->mapped_here = true;
  return true;
}

void release_source(emelb_window* w) {
  if (w->locked_base) cudaHostUnregister(w->locked_base);
  if (w->mapped_here && w->source) ::munmap(const_cast<uint8_t*>(w->source), size_t(w->source_bytes));
  cudaGetLastError();
  w->page_locked = false;
  w->locked_base = nullptr;
  w->mapped_here = false;
  w->source = nullptr;
  w->source_bytes = 0;
}

// page-lock the pages the extents lie in, read-only: the copy engines then read the source in place
bool lock_source(emelb_window* w) {
  cudaPointerAttributes at{};
  if (cudaPointerGetAttributes(&at, w->source) == cudaSuccess && at.type == cudaMemoryTypeHost) return true;   // already is: nothing to undo
  cudaGetLastError();
  uint64_t lo = ~0ull, hi = 0;
  for (const emelb_window_layer& d : w->plan) {
    lo = d.file_begin < lo ? d.file_begin : lo;
    hi = d.file_begin + d.file_span > hi ? d.file_begin + d.file_span : hi;
  }
  const uintptr_t page = uintptr_t(sysconf(_SC_PAGESIZE));
  const uintptr_t a = (uintptr_t(w->source) + lo) & ~(page - 1);
  const uintptr_t b = (uintptr_t(w->source) + hi + page - 1) & ~(page - 1);
  // read-only first (the only form a PROT_READ mapping takes), then the plain form for ordinary memory
  if (cudaHostRegister(reinterpret_cast<void*>(a), b - a, cudaHostRegisterReadOnly) != cudaSuccess) {
    cudaGetLastError();
    if (w->mapped_here || cudaHostRegister(reinterpret_cast<void*>(a), b - a, cudaHostRegisterDefault) != cudaSuccess) {
      cudaGetLastError();
      return false;
    }
  }
  w->locked_base = reinterpret_cast<void*>(a);
  return true;
}

bool take_injected_failure(emelb_window* w) {
  if (w->fail_next <= 0) return false;
  --w->fail_next;
  return true;
}

// staged route: one extent through the two page-locked buffers, chunk by chunk
bool stage_extent(emelb_window* w, uint8_t* dst, const uint8_t* src, uint64_t bytes, int& turn) {
  for (uint64_t at = 0; at < bytes; at += w->chunk, turn ^= 1) {
    const uint64_t n = bytes - at < w->chunk ? bytes - at : w->chunk;
    if (cudaEventSynchronize(w->drained[turn]) != cudaSuccess) return false;   // the copy that last read this buffer
    std::memcpy(w->pinned[turn], src + at, size_t(n));
    if (cudaMemcpyAsync(dst + at, w->pinned[turn], size_t(n), cudaMemcpyHostToDevice, w->copy_stream) != cudaSuccess) return false;
    if (cudaEventRecord(w->drained[turn], w->copy_stream) != cudaSuccess) return false;
  }
  return true;
}

void worker_body(emelb_window* w) {
  cudaSetDevice(w->c->device);
  int turn = 0;
  for (;;) {
    int si = -1, layer = -1;
    bool injected = false;
    {
      std::unique_lock<std::mutex> lk(w->m);
      w->cv.wait(lk, [&] { return w->stop || !w->jobs.empty(); });
      if (w->jobs.empty()) return;   // stop, queue drained
      si = w->jobs.front();
      w->jobs.pop_front();
      w->busy = true;
      layer = w->slots[si].layer;
      injected = take_injected_failure(w);
    }
    Slot& slot = w->slots[si];
    const emelb_window_layer& d = w->plan[size_t(layer)];
    bool ok = !injected && cudaEventSynchronize(slot.released) == cudaSuccess;   // the slot's previous readers have run
    uint64_t copied = 0;
    for (uint32_t i = 0; ok && i < d.weight_count; ++i) {
      const emelb_window_extent& e = d.weights[i];
      ok = stage_extent(w, slot.storage + e.slot_offset, w->source + e.file_offset, e.byte_size, turn);
      copied += e.byte_size;
    }
    ok = ok && cudaStreamSynchronize(w->copy_stream) == cudaSuccess;
    if (!ok) cudaGetLastError();
    {
      std::lock_guard<std::mutex> lk(w->m);
      slot.lifecycle = ok ? RESIDENT : FAILED;
      if (ok) w->stats.bytes_copied += copied;
      else ++w->stats.loads_failed;
      w->busy = false;
    }
    w->cv.notify_all();
  }
}

// detail: bind_and_submit_layer_load of the reference (actions.hpp:27-60).  Caller holds no lock.
void submit_load(emelb_window* w, int layer) {
  const int si = int(uint32_t(layer) % w->slot_count);
  Slot& slot = w->slots[si];
  ++w->stats.loads_submitted;
  if (!w->page_locked) {
    {
      std::lock_guard<std::mutex> lk(w->m);
      slot.layer = layer;
      slot.lifecycle = LOADING;
      w->jobs.push_back(si);
    }
    w->cv.notify_all();
    return;
  }
  slot.layer = layer;
  const emelb_window_layer& d = w->plan[size_t(layer)];
  bool ok = !take_injected_failure(w);
  ok = ok && cudaStreamWaitEvent(w->copy_stream, slot.released, 0) == cudaSuccess;
  uint64_t copied = 0;
  for (uint32_t i = 0; ok && i < d.weight_count; ++i) {
    const emelb_window_extent& e = d.weights[i];
    ok = cudaMemcpyAsync(slot.storage + e.slot_offset, w->source + e.file_offset, size_t(e.byte_size), cudaMemcpyHostToDevice,
                         w->copy_stream) == cudaSuccess;
    copied += e.byte_size;
  }
  ok = ok && cudaEventRecord(slot.loaded, w->copy_stream) == cudaSuccess;
  if (!ok) {
    cudaGetLastError();
    ++w->stats.loads_failed;
  } else {
    w->stats.bytes_copied += copied;
  }
  slot.lifecycle = ok ? RESIDENT : FAILED;   // resident in stream order: readers wait for `loaded`
}

// wait on the host until the staged route has finished with slot si (no-op on the page-locked route)
void join_slot(emelb_window* w, int si) {
  if (w->page_locked) return;
  std::unique_lock<std::mutex> lk(w->m);
  w->cv.wait(lk, [&] { return w->slots[si].lifecycle != LOADING; });
}

int slot_state(emelb_window* w, int si) {
  std::lock_guard<std::mutex> lk(w->m);
  return w->slots[si].lifecycle;
}

void join_all(emelb_window* w) {
  if (w->worker.joinable()) {
    std::unique_lock<std::mutex> lk(w->m);
    w->cv.wait(lk, [&] { return w->jobs.empty() && !w->busy; });
  }
  if (w->copy_stream) cudaStreamSynchronize(w->copy_stream);
  cudaGetLastError();
}

void stop_worker(emelb_window* w) {
  if (!w->worker.joinable()) return;
  {
    std::lock_guard<std::mutex> lk(w->m);
    w->stop = true;
  }
  w->cv.notify_all();
  w->worker.join();
  w->stop = false;
}

void release_staging(emelb_window* w) {
  for (int i = 0; i < 2; ++i) {
    if (w->drained[i]) cudaEventDestroy(w->drained[i]);
    if (w->pinned[i]) cudaFreeHost(w->pinned[i]);
    w->drained[i] = nullptr;
    w->pinned[i] = nullptr;
  }
}

void reset_window(emelb_window* w) {
  for (Slot& s : w->slots) {
    s.storage = nullptr;
    s.layer = -1;
    s.lifecycle = VACANT;
  }
  w->plan.clear();
  w->slot_count = 0;
  w->slot_capacity = 0;
  w->published_slot = -1;
  w->streaming = false;
  w->bound = false;
}

bool device_pointer(const void* p, int device) {
  cudaPointerAttributes at{};
  if (cudaPointerGetAttributes(&at, p) != cudaSuccess) {
    cudaGetLastError();
    return false;
  }
  return at.type == cudaMemoryTypeDevice && at.device == device;
}

// The decisions of a bind once the plan is known (guards.hpp:83-186): a zero budget or a model that fits binds as
// passthrough; else slot / prefetch sizing, then the slots against the budget, then the storage.  device < 0: the
// storage is not asked of the CUDA runtime (a request checked on a host without a GPU)
uint32_t budget_decision(const emelb_window_request& r, uint64_t slot_capacity, uint64_t total, int device, bool* fits) {
  *fits = r.budget_bytes == 0 || total <= r.budget_bytes;
  if (*fits) return EMELB_WINDOW_OK;
  const bool config = r.window_slots >= 2 && r.window_slots <= EMELB_WINDOW_MAX_SLOTS && r.prefetch_depth > 0 &&
                      r.prefetch_depth < r.window_slots;
  const uint64_t need = uint64_t(r.window_slots) * slot_capacity;
  if (!config) return EMELB_WINDOW_INVALID_REQUEST;
  if (need > r.budget_bytes) return EMELB_WINDOW_BUDGET_TOO_SMALL;
  if (!r.slot_storage || r.slot_storage_bytes < need ||
      (reinterpret_cast<uintptr_t>(r.slot_storage) % EMELB_WINDOW_SLOT_ALIGNMENT) != 0 ||
      (device >= 0 && !device_pointer(r.slot_storage, device)))
    return EMELB_WINDOW_SLOT_STORAGE_TOO_SMALL;
  return EMELB_WINDOW_OK;
}

uint32_t do_unbind(emelb_window* w) {
  if (!w->bound) return EMELB_WINDOW_NOT_BOUND;
  cudaSetDevice(w->c->device);
  join_all(w);
  cudaStreamSynchronize(w->c->stream);   // work that reads a slot has run: the caller may free the storage
  cudaGetLastError();
  stop_worker(w);
  release_staging(w);
  release_source(w);
  reset_window(w);
  return EMELB_WINDOW_OK;
}

}  // namespace

namespace emelb {

bool window_streaming(const emelb_window* w) { return w && w->bound && w->streaming; }
emelb_ctx* window_ctx(const emelb_window* w) { return w ? w->c : nullptr; }
int window_layer_count(const emelb_window* w) { return w ? int(w->plan.size()) : 0; }

bool window_find_extent(const emelb_window* w, int layer, const void* host, uint64_t bytes, uint64_t* slot_offset) {
  if (!window_streaming(w) || layer < 0 || size_t(layer) >= w->plan.size()) return false;
  const uint8_t* p = static_cast<const uint8_t*>(host);
  if (p < w->source || p >= w->source + w->source_bytes) return false;
  const uint64_t off = uint64_t(p - w->source);
  const emelb_window_layer& d = w->plan[size_t(layer)];
  for (uint32_t i = 0; i < d.weight_count; ++i)
    if (d.weights[i].file_offset == off && d.weights[i].byte_size == bytes) {
      *slot_offset = d.weights[i].slot_offset;
      return true;
    }
  return false;
}

}  // namespace emelb

extern "C" {

uint32_t emelb_window_create(emelb_ctx* ctx, emelb_window** out) {
  if (!ctx || !out) return EMELB_WINDOW_INVALID_REQUEST;
  *out = nullptr;
  emelb_window* w = new (std::nothrow) emelb_window();
  if (!w) return EMELB_WINDOW_INTERNAL_ERROR;
  w->c = ctx;
  cudaSetDevice(ctx->device);
  bool ok = cudaStreamCreateWithFlags(&w->copy_stream, cudaStreamNonBlocking) == cudaSuccess;
  for (Slot& s : w->slots)
    ok = ok && cudaEventCreateWithFlags(&s.loaded, cudaEventDisableTiming) == cudaSuccess &&
         cudaEventCreateWithFlags(&s.released, cudaEventDisableTiming) == cudaSuccess;
  if (!ok) {
    cudaGetLastError();
    emelb_window_destroy(w);
    return EMELB_WINDOW_INTERNAL_ERROR;
  }
  *out = w;
  return EMELB_WINDOW_OK;
}

uint32_t emelb_window_destroy(emelb_window* w) {
  if (!w) return EMELB_WINDOW_INVALID_REQUEST;
  cudaSetDevice(w->c->device);
  if (w->bound) do_unbind(w);
  for (Slot& s : w->slots) {
    if (s.loaded) cudaEventDestroy(s.loaded);
    if (s.released) cudaEventDestroy(s.released);
  }
  if (w->copy_stream) cudaStreamDestroy(w->copy_stream);
  cudaGetLastError();
  delete w;
  return EMELB_WINDOW_OK;
}

uint32_t emelb_window_bind(emelb_window* w, const emelb_window_request* request, emelb_window_bound* out) {
  if (!w || !request) return EMELB_WINDOW_INVALID_REQUEST;
  if (out) *out = emelb_window_bound{};
  if (w->bound) return EMELB_WINDOW_ALREADY_BOUND;
  const emelb_window_request& r = *request;
  if (!request_valid(r)) return EMELB_WINDOW_INVALID_REQUEST;
  cudaSetDevice(w->c->device);
  if (!map_source(w, r)) return EMELB_WINDOW_SOURCE_MAP_FAILED;
  scan_layers(w, r);
  uint64_t total = 0;
  for (const emelb_window_layer& d : w->plan) total += d.slot_bytes;
  bool fits = false;
  const uint32_t err = budget_decision(r, w->slot_capacity, total, w->c->device, &fits);
  if (err != EMELB_WINDOW_OK) {
    release_source(w);
    reset_window(w);
    return err;
  }
  w->stats = emelb_window_stats{};
  w->bound = true;
  w->streaming = !fits;
  w->prefetch_depth = r.prefetch_depth;
  w->chunk = r.stage_chunk_bytes;
  if (w->streaming) {
    w->slot_count = r.window_slots;
    for (uint32_t i = 0; i < w->slot_count; ++i) w->slots[i].storage = static_cast<uint8_t*>(r.slot_storage) + uint64_t(i) * w->slot_capacity;
    w->page_locked = !w->staged_only && lock_source(w);
    if (!w->page_locked) {
      bool ok = true;
      for (int i = 0; i < 2 && ok; ++i)
        ok = cudaHostAlloc(&w->pinned[i], size_t(w->chunk), cudaHostAllocDefault) == cudaSuccess &&
             cudaEventCreateWithFlags(&w->drained[i], cudaEventDisableTiming) == cudaSuccess;
      if (ok) {
        try {
          w->worker = std::thread(worker_body, w);
        } catch (...) {
          ok = false;
        }
      }
      if (!ok) {
        cudaGetLastError();
        release_staging(w);
        release_source(w);
        reset_window(w);
        return EMELB_WINDOW_INTERNAL_ERROR;
      }
    }
    // actions.hpp:218-227: prime the ring with the first prefetch_depth layers
    const uint32_t depth = w->prefetch_depth < uint32_t(w->plan.size()) ? w->prefetch_depth : uint32_t(w->plan.size());
    for (uint32_t l = 0; l < depth; ++l) submit_load(w, int(l));
  }
  if (out) {
    out->streaming_active = w->streaming ? 1 : 0;
    out->source_base = w->source;
    out->source_bytes = w->source_bytes;
    out->window_slots = w->slot_count;
    out->source_page_locked = w->page_locked ? 1 : 0;
  }
  return EMELB_WINDOW_OK;
}

uint32_t emelb_window_check(const emelb_window_request* request, int32_t* streaming_active, uint64_t* slot_capacity_bytes,
                            uint64_t* total_bytes) {
  if (!request) return EMELB_WINDOW_INVALID_REQUEST;
  if (streaming_active) *streaming_active = 0;
  if (!request_valid(*request)) return EMELB_WINDOW_INVALID_REQUEST;
  if (request->file_size_bytes > kMaxMappingBytes) return EMELB_WINDOW_SOURCE_MAP_FAILED;
  emelb_window plan;   // holds the scanned plan only; no device object is touched
  scan_layers(&plan, *request);
  uint64_t total = 0;
  for (const emelb_window_layer& d : plan.plan) total += d.slot_bytes;
  if (slot_capacity_bytes) *slot_capacity_bytes = plan.slot_capacity;
  if (total_bytes) *total_bytes = total;
  bool fits = false;
  const uint32_t err = budget_decision(*request, plan.slot_capacity, total, -1, &fits);
  if (err == EMELB_WINDOW_OK && streaming_active) *streaming_active = fits ? 0 : 1;
  return err;
}

uint32_t emelb_window_acquire(emelb_window* w, int32_t layer_index, const uint8_t** slot_base, const emelb_window_layer** layout) {
  if (!w) return EMELB_WINDOW_INVALID_REQUEST;
  if (slot_base) *slot_base = nullptr;
  if (layout) *layout = nullptr;
  if (!w->bound) return EMELB_WINDOW_NOT_BOUND;
  if (!w->streaming) return EMELB_WINDOW_NOT_STREAMING;
  if (layer_index < 0 || size_t(layer_index) >= w->plan.size()) return EMELB_WINDOW_LAYER_OUT_OF_RANGE;
  cudaSetDevice(w->c->device);
  ++w->stats.acquires;
  // the view handed out before ends here: everything that reads it is on the compute stream by now
  if (w->published_slot >= 0 && cudaEventRecord(w->slots[w->published_slot].released, w->c->stream) != cudaSuccess) {
    cudaGetLastError();
    return EMELB_WINDOW_INTERNAL_ERROR;
  }
  const int si = int(uint32_t(layer_index) % w->slot_count);
  Slot& slot = w->slots[si];
  // guards.hpp:310-322: a slot still loading another layer is joined before it is reused.  slot.layer is written by
  // this thread only; the lifecycle is shared with the I/O thread and read under the lock
  if (slot.layer != layer_index) join_slot(w, si);
  if (slot.layer == layer_index) {
    ++w->stats.acquires_resident;
  } else {
    ++w->stats.acquires_cold;
    submit_load(w, layer_index);
  }
  join_slot(w, si);
  if (slot_state(w, si) == FAILED) {
    // guards.hpp:386-398: one more try before the error is reported
    submit_load(w, layer_index);
    join_slot(w, si);
  }
  if (slot_state(w, si) != RESIDENT) return EMELB_WINDOW_SLOT_COPY_FAILED;
  if (w->page_locked && cudaStreamWaitEvent(w->c->stream, slot.loaded, 0) != cudaSuccess) {
    cudaGetLastError();
    return EMELB_WINDOW_INTERNAL_ERROR;
  }
  w->published_slot = si;
  // guards.hpp:433-452: advance the ring, never into the slot just handed out
  const int ahead = int((uint32_t(layer_index) + w->prefetch_depth) % uint32_t(w->plan.size()));
  const int ti = int(uint32_t(ahead) % w->slot_count);
  if (ti != si) {
    bool idle;
    {
      std::lock_guard<std::mutex> lk(w->m);
      idle = w->slots[ti].layer != ahead && w->slots[ti].lifecycle != LOADING;
    }
    if (idle) submit_load(w, ahead);
  }
  if (slot_base) *slot_base = slot.storage;
  if (layout) *layout = &w->plan[size_t(layer_index)];
  return EMELB_WINDOW_OK;
}

uint32_t emelb_window_unbind(emelb_window* w) {
  if (!w) return EMELB_WINDOW_INVALID_REQUEST;
  return do_unbind(w);
}

uint32_t emelb_window_get_stats(const emelb_window* w, emelb_window_stats* out) {
  if (!w || !out) return EMELB_WINDOW_INVALID_REQUEST;
  std::lock_guard<std::mutex> lk(const_cast<emelb_window*>(w)->m);
  *out = w->stats;
  return EMELB_WINDOW_OK;
}

uint32_t emelb_window_layer_plan(const emelb_window* w, int32_t layer_index, const emelb_window_layer** out, uint64_t* slot_capacity_bytes) {
  if (!w || !out) return EMELB_WINDOW_INVALID_REQUEST;
  *out = nullptr;
  if (!w->bound) return EMELB_WINDOW_NOT_BOUND;
  if (layer_index < 0 || size_t(layer_index) >= w->plan.size()) return EMELB_WINDOW_LAYER_OUT_OF_RANGE;
  *out = &w->plan[size_t(layer_index)];
  if (slot_capacity_bytes) *slot_capacity_bytes = w->slot_capacity;
  return EMELB_WINDOW_OK;
}

uint32_t emelb_window_fail_next_loads(emelb_window* w, int32_t count) {
  if (!w || count < 0) return EMELB_WINDOW_INVALID_REQUEST;
  std::lock_guard<std::mutex> lk(w->m);
  w->fail_next = count;
  return EMELB_WINDOW_OK;
}

uint32_t emelb_window_set_staged_only(emelb_window* w, int32_t staged_only) {
  if (!w) return EMELB_WINDOW_INVALID_REQUEST;
  if (w->bound) return EMELB_WINDOW_ALREADY_BOUND;
  w->staged_only = staged_only != 0;
  return EMELB_WINDOW_OK;
}

}  // extern "C"
