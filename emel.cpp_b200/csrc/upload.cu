// Host span -> HBM for the residency table.
//
// A weight span usually lies in a file mapping (page cache), which the copy
// engines cannot read directly.  Three routes, picked per call:
//   * spans that are already page-locked, and small spans: one cudaMemcpyAsync;
//   * EMELB_UPLOAD_MODE=register: page-lock the span read-only in place, one DMA
//     straight from the page cache, unlock (no intermediate copy at all);
//   * default: several threads each walk their share of the span in 4 MB chunks
//     through two page-locked buffers of their own -- filling one chunk overlaps
//     the DMA of the previous one, and the threads overlap each other.  A chunk
//     is filled by pread() when the caller names the file the span maps (the
//     kernel copies out of the page cache without touching this process's page
//     tables), else by memcpy from the span (one page fault per fresh page).
// Bytes arrive unchanged; the call returns when the whole span is in HBM.
#include <unistd.h>

#include <algorithm>
#include <atomic>
#include <cerrno>
#include <cstdlib>
#include <cstring>
#include <thread>
#include <vector>

#include "ctx.h"

namespace emelb {

namespace {

constexpr uint64_t kChunk = 4ull << 20;
constexpr uint64_t kDirectBelow = 4ull << 20;
constexpr int kMaxUploadThreads = 16;

int upload_threads(const emelb_ctx* c) {
  int n = int(std::min<unsigned>(16u, std::max(1u, std::thread::hardware_concurrency())));
  if (c->upload_threads > 0) n = c->upload_threads;
  return std::max(1, std::min(n, kMaxUploadThreads));
}

bool page_locked(const void* p) {
  cudaPointerAttributes a{};
  if (cudaPointerGetAttributes(&a, p) != cudaSuccess) {
    cudaGetLastError();
    return false;
  }
  return a.type == cudaMemoryTypeHost;
}

// the read-only in-place route; false = not available here, nothing was copied
bool upload_registered(emelb_ctx* c, void* dev, const void* host, uint64_t bytes) {
  if (bytes < kDirectBelow) return false;
  const uintptr_t page = uintptr_t(sysconf(_SC_PAGESIZE));
  const uintptr_t lo = uintptr_t(host) & ~(page - 1);
  const uintptr_t hi = (uintptr_t(host) + bytes + page - 1) & ~(page - 1);
  if (cudaHostRegister(reinterpret_cast<void*>(lo), hi - lo, cudaHostRegisterReadOnly) != cudaSuccess) {
    cudaGetLastError();
    return false;
  }
  cudaError_t e = cudaMemcpyAsync(dev, host, bytes, cudaMemcpyHostToDevice, c->stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(c->stream);
  cudaHostUnregister(reinterpret_cast<void*>(lo));
  if (e != cudaSuccess) c->last_cuda_error = int(e);
  return e == cudaSuccess;
}

}  // namespace

bool upload_ring_reserve(emelb_ctx* c, int threads) {
  while (int(c->upload_lanes.size()) < threads) {
    UploadLane lane;
    bool ok = cudaStreamCreateWithFlags(&lane.stream, cudaStreamNonBlocking) == cudaSuccess;
    for (int s = 0; s < 2 && ok; ++s) {
      ok = cudaHostAlloc(&lane.pinned[s], kChunk, cudaHostAllocDefault) == cudaSuccess &&
           cudaEventCreateWithFlags(&lane.drained[s], cudaEventDisableTiming) == cudaSuccess;
    }
    c->upload_lanes.push_back(lane);  // kept even when incomplete, so that release frees what exists
    if (!ok) {
      cudaGetLastError();
      return false;
    }
  }
  return true;
}

void upload_ring_release(emelb_ctx* c) {
  for (UploadLane& lane : c->upload_lanes) {
    for (int s = 0; s < 2; ++s) {
      if (lane.drained[s]) cudaEventDestroy(lane.drained[s]);
      if (lane.pinned[s]) cudaFreeHost(lane.pinned[s]);
    }
    if (lane.stream) cudaStreamDestroy(lane.stream);
  }
  c->upload_lanes.clear();
}

cudaError_t upload_spans(emelb_ctx* c, const UploadSpan* spans, size_t count, int fd) {
  const bool want_register = c->upload_route == EMELB_UPLOAD_REGISTER;
  const bool want_plain = c->upload_route == EMELB_UPLOAD_PLAIN;
  // spans that go in one copy; the rest is cut into chunks for the lanes
  struct Chunk {
    void* dev;
    const uint8_t* host;
    uint64_t file_offset, bytes;
  };
  std::vector<Chunk> chunks;
  for (size_t i = 0; i < count; ++i) {
    const UploadSpan& sp = spans[i];
    if (sp.bytes == 0) continue;
    const bool direct = want_plain || page_locked(sp.host) || (sp.bytes < kDirectBelow && count == 1);
    if (want_register && upload_registered(c, sp.dev, sp.host, sp.bytes)) continue;
    if (direct) {
      cudaError_t e = cudaMemcpyAsync(sp.dev, sp.host, sp.bytes, cudaMemcpyHostToDevice, c->stream);
      if (e == cudaSuccess) e = cudaStreamSynchronize(c->stream);
      if (e != cudaSuccess) return e;
      continue;
    }
    for (uint64_t at = 0; at < sp.bytes; at += kChunk)
      chunks.push_back(Chunk{static_cast<uint8_t*>(sp.dev) + at, static_cast<const uint8_t*>(sp.host) + at,
                             sp.file_offset + at, std::min(kChunk, sp.bytes - at)});
  }
  if (chunks.empty()) return cudaSuccess;

  const int threads = int(std::min<uint64_t>(uint64_t(upload_threads(c)), chunks.size()));
  if (!upload_ring_reserve(c, threads)) return cudaErrorMemoryAllocation;
  std::atomic<int> first_error{int(cudaSuccess)};
  auto fill = [&](void* dst, const Chunk& ch) {
    if (fd < 0) {
      std::memcpy(dst, ch.host, ch.bytes);
      return true;
    }
    uint64_t got = 0;
    while (got < ch.bytes) {
      const ssize_t r = ::pread(fd, static_cast<uint8_t*>(dst) + got, ch.bytes - got, off_t(ch.file_offset + got));
      if (r < 0 && errno == EINTR) continue;
      if (r <= 0) return false;
      got += uint64_t(r);
    }
    return true;
  };
  auto lane_body = [&](int t) {
    UploadLane& lane = c->upload_lanes[t];
    cudaError_t e = cudaSetDevice(c->device);
    int turn = 0;
    // chunk i belongs to lane i % threads: neighbouring chunks are read concurrently
    for (size_t i = size_t(t); i < chunks.size() && e == cudaSuccess; i += size_t(threads), turn ^= 1) {
      const Chunk& ch = chunks[i];
      e = cudaEventSynchronize(lane.drained[turn]);  // the DMA that last read this buffer (done at once the first time)
      if (e != cudaSuccess) break;
      if (!fill(lane.pinned[turn], ch)) {
        e = cudaErrorUnknown;  // the file ended or failed under the mapping
        break;
      }
      e = cudaMemcpyAsync(ch.dev, lane.pinned[turn], ch.bytes, cudaMemcpyHostToDevice, lane.stream);
      if (e == cudaSuccess) e = cudaEventRecord(lane.drained[turn], lane.stream);
    }
    const cudaError_t done = cudaStreamSynchronize(lane.stream);
    if (e == cudaSuccess) e = done;
    if (e != cudaSuccess) {
      int expected = int(cudaSuccess);
      first_error.compare_exchange_strong(expected, int(e));
    }
  };
  std::vector<std::thread> workers;
  std::vector<int> inline_lanes{0};
  workers.reserve(size_t(threads));
  for (int t = 1; t < threads; ++t) {
    try {
      workers.emplace_back(lane_body, t);
    } catch (...) {
      inline_lanes.push_back(t);  // no thread to be had: this lane's chunks are copied by the caller
    }
  }
  for (int t : inline_lanes) lane_body(t);
  for (std::thread& w : workers) w.join();
  return cudaError_t(first_error.load());
}

}  // namespace emelb
