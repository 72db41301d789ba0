// emelb_mul_mat_vec_noalloc — the quantized mat-vec for callers that must not
// allocate.
//
// Some code that wants this kernel runs where device allocation is off limits:
// a real-time serving loop whose latency budget forbids the implicit device
// synchronisation of cudaMalloc/cudaFree, a host callback or driver-adjacent
// hook in which allocating is not allowed, or a process whose device memory is
// owned by someone else's pool and already sized to the last byte.  emelb_create cannot
// serve them (it allocates its workspace).  This entry point needs no context
// at all: the mat-vec's scratch — the quantized activation planes and the task
// counter of the streaming kernel — lives in a fixed array that is part of the
// loaded library image, so every GPU that loads the library carries
// kNoAllocScratchBytes of it until the process exits, and nothing is allocated
// or freed here, by this file or by anything it calls.
//
// Limits and rules that follow from the fixed array:
//  * K (the row length) is at most kNoAllocMaxK; larger requests are refused.
//  * All calls on one device share the array.  It still holds the previous
//    call's activations; this call overwrites the part it uses and clears the
//    task counter itself.  Two calls that overlap on the GPU (different streams,
//    or two host threads) race on it — serialise them.
//  * The first call on each device looks up the array's device address (a host
//    side step, done once per device with that device current).  Make that
//    first call outside any stream capture.
//  * The calling thread's current device is the same after the call as before it.
//  * There is no context to report through, so a copy wait that ran out inside
//    the kernel (the bounded waits of the streaming kernel) is not reported: the
//    kernel raises a word in the scratch array that stays raised, nothing reads it.
#include <atomic>
#include <cstdio>
#include <cstring>

#include "../../include/emelb.h"
#include "ctx.h"

using namespace emelb;

namespace {

constexpr int kNoAllocMaxK = 32768;  // = 128 Q8_K blocks / 1024 Q8_0 blocks, the reference's own limits
// planes: qs[K] int8 | d[K/32] f32 (covers K/256 too) | bsums[K/16] int16 | task counter (2 ints, padded)
constexpr size_t kQsBytes = kNoAllocMaxK;
constexpr size_t kDBytes = kNoAllocMaxK / 32 * sizeof(float);
constexpr size_t kBsBytes = kNoAllocMaxK / 16 * sizeof(int16_t);
constexpr size_t kSchedBytes = 256;
constexpr size_t kNoAllocScratchBytes = kQsBytes + kDBytes + kBsBytes + kSchedBytes;  // 41,216 B

// In host code this name is only a handle for the runtime (its value is not a
// device address); the address the kernels get comes from cudaGetSymbolAddress.
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocScratchBytes];

constexpr int kMaxDevices = 64;
// the address is published last, with release order: a thread that sees it also sees the SM count
std::atomic<unsigned char*> g_scratch_addr[kMaxDevices] = {};
int g_sm_count[kMaxDevices] = {};

// makes `device` current for the call and puts the caller's device back on every return path
struct DeviceScope {
  int previous = -1;
  bool ok = false;
  explicit DeviceScope(int device) {
    if (cudaGetDevice(&previous) != cudaSuccess) previous = -1;
    ok = cudaSetDevice(device) == cudaSuccess;
  }
  ~DeviceScope() {
    if (previous >= 0) cudaSetDevice(previous);
    cudaGetLastError();
  }
};

void explain(char* text, uint64_t bytes, const char* msg) {
  if (text && bytes) {
    std::snprintf(text, (size_t)bytes, "%s", msg);
  }
}

uint32_t refuse(char* text, uint64_t bytes, const char* msg) {
  explain(text, bytes, msg);
  return EMELB_INVALID_REQUEST;
}

}  // namespace

extern "C" uint32_t emelb_mul_mat_vec_noalloc(int device, void* stream, int32_t weight_type, const void* weights_dev,
                                              uint64_t k, uint64_t m, const float* x_dev, float* y_dev, char* error_text,
                                              uint64_t error_text_bytes) {
  explain(error_text, error_text_bytes, "");
  const bool quant = weight_type == T_Q4_K || weight_type == T_Q6_K || weight_type == T_Q8_0 || weight_type == T_Q4_0;
  if (!quant) return refuse(error_text, error_text_bytes, "weight_type must be Q4_K, Q6_K, Q8_0 or Q4_0");
  if (!weights_dev || !x_dev || !y_dev) return refuse(error_text, error_text_bytes, "null operand pointer");
  if (device < 0 || device >= kMaxDevices) return refuse(error_text, error_text_bytes, "device index out of range");
  const uint64_t be = (uint64_t)block_elems(weight_type);
  if (k == 0 || m == 0 || k % be != 0) return refuse(error_text, error_text_bytes, "K must be a non-zero multiple of the block size");
  if (k > (uint64_t)kNoAllocMaxK) {
    char msg[160];
    std::snprintf(msg, sizeof msg, "K = %llu exceeds the fixed scratch of this entry point (K <= %d)", (unsigned long long)k,
                  kNoAllocMaxK);
    return refuse(error_text, error_text_bytes, msg);
  }
  if (m > 0x7fffffffull) return refuse(error_text, error_text_bytes, "row count out of range");

  DeviceScope scope(device);
  if (!scope.ok) {
    cudaGetLastError();
    explain(error_text, error_text_bytes, "cudaSetDevice failed");
    return EMELB_INTERNAL_ERROR;
  }
  if (!g_scratch_addr[device].load(std::memory_order_acquire)) {
    // once per device, with that device current
    void* p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
    cudaDeviceProp prop{};
    if (e != cudaSuccess || !p || cudaGetDeviceProperties(&prop, device) != cudaSuccess) {
      cudaGetLastError();
      explain(error_text, error_text_bytes, "cudaGetSymbolAddress failed for the scratch array");
      return EMELB_INTERNAL_ERROR;
    }
    g_sm_count[device] = prop.multiProcessorCount;
    g_scratch_addr[device].store(static_cast<unsigned char*>(p), std::memory_order_release);
  }
  unsigned char* base = g_scratch_addr[device].load(std::memory_order_acquire);
  cudaStream_t st = static_cast<cudaStream_t>(stream);

  ActPlanesMut planes{};
  planes.qs = reinterpret_cast<int8_t*>(base);
  planes.d = reinterpret_cast<float*>(base + kQsBytes);
  planes.bsums = reinterpret_cast<int16_t*>(base + kQsBytes + kDBytes);
  int* sched = reinterpret_cast<int*>(base + kQsBytes + kDBytes + kBsBytes);

  // the task counter (two ints) must start at zero whatever the previous call left behind; the word after
  // it is the kernel's "a wait ran out" mark and is left alone
  cudaError_t e = cudaMemsetAsync(sched, 0, 2 * sizeof(int), st);
  if (e == cudaSuccess) e = quantize_into_planes(weight_type, x_dev, 1, 1, (int)k, planes, st);
  if (e == cudaSuccess) {
    GemvArgs a{};
    a.W = static_cast<const uint8_t*>(weights_dev);
    a.row_bytes = (int64_t)(k / be) * block_bytes(weight_type);
    a.M = (int)m;
    a.K = (int)k;
    a.act = planes_view(planes, weight_type, (int)k);
    a.col0 = 0;
    a.y = y_dev;
    a.ldy = 1;
    a.residual = nullptr;
    a.sched = sched;
    a.status = sched + 2;
    int launches = 0;
    e = launch_gemv(weight_type, a, 1, false, g_sm_count[device], st, &launches);
  }
  if (e != cudaSuccess) {
    cudaGetLastError();
    explain(error_text, error_text_bytes, cudaGetErrorString(e));
    return EMELB_INTERNAL_ERROR;
  }
  return EMELB_OK;
}
