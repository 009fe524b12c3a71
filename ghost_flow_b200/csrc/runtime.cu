// Device layer behind a C ABI: device queries, streams, events, a timer, an error table and a pooled device
// allocator with size classes and usage statistics.
//
// Counterparts in the reference: ghostflow-cuda/src/device.rs (properties, capability predicates), stream.rs
// (streams, events, timers), memory.rs (GpuMemoryPool with power-of-two classes, current/peak usage), error.rs
// (error enum). The reference's copies are no-ops and its stream waits synchronise the host; these call the
// CUDA runtime for real. Handles are opaque pointers; every function returns 0 on success or a GFRT_* code.
#include <cuda_runtime.h>

#include <cstdint>
#include <cstring>
#include <map>
#include <mutex>
#include <vector>

#include "gf_host.h"

namespace {

enum GfrtError : int {
  GFRT_OK = 0,
  GFRT_NOT_AVAILABLE = 1,
  GFRT_INVALID_DEVICE = 2,
  GFRT_OUT_OF_MEMORY = 3,
  GFRT_LAUNCH_FAILURE = 4,
  GFRT_INVALID_VALUE = 5,
  GFRT_NOT_READY = 6,
  GFRT_UNKNOWN = 99,
};

int map_error(cudaError_t e) {
  switch (e) {
    case cudaSuccess: return GFRT_OK;
    case cudaErrorNoDevice:
    case cudaErrorInsufficientDriver: return GFRT_NOT_AVAILABLE;
    case cudaErrorInvalidDevice: return GFRT_INVALID_DEVICE;
    case cudaErrorMemoryAllocation: return GFRT_OUT_OF_MEMORY;
    case cudaErrorLaunchFailure: return GFRT_LAUNCH_FAILURE;
    case cudaErrorInvalidValue: return GFRT_INVALID_VALUE;
    case cudaErrorNotReady: return GFRT_NOT_READY;
    default: return GFRT_UNKNOWN;
  }
}

struct Pool {
  int device;
  std::mutex mu;
  std::map<size_t, std::vector<void*>> free_lists;   // size class -> cached blocks
  std::map<void*, size_t> live;                      // block -> size class
  size_t current = 0, peak = 0, cached = 0;
  uint64_t hits = 0, misses = 0;
};

size_t size_class(size_t n) {
  size_t c = 256;
  while (c < n) c <<= 1;
  return c;
}

}  // namespace

struct GfrtProps {
  char name[256];
  int major, minor, multiprocessors, warp_size, max_threads_per_block, clock_khz, memory_clock_khz;
  int l2_bytes, max_shared_per_block_optin;
  unsigned long long total_memory;
};

GF_API const char* gfrt_error_string(int code) {
  switch (code) {
    case GFRT_OK: return "success";
    case GFRT_NOT_AVAILABLE: return "cuda is not available";
    case GFRT_INVALID_DEVICE: return "invalid device ordinal";
    case GFRT_OUT_OF_MEMORY: return "out of memory";
    case GFRT_LAUNCH_FAILURE: return "kernel launch failed";
    case GFRT_INVALID_VALUE: return "invalid value";
    case GFRT_NOT_READY: return "not ready";
    default: return "unknown error";
  }
}

GF_API int gfrt_device_count(int* n) {
  cudaError_t e = cudaGetDeviceCount(n);
  if (e != cudaSuccess) *n = 0;
  return map_error(e);
}

GF_API int gfrt_device_props(int device, GfrtProps* out) {
  cudaDeviceProp p;
  cudaError_t e = cudaGetDeviceProperties(&p, device);
  if (e != cudaSuccess) return map_error(e);
  std::memset(out, 0, sizeof(*out));
  std::strncpy(out->name, p.name, sizeof(out->name) - 1);
  out->major = p.major; out->minor = p.minor; out->multiprocessors = p.multiProcessorCount;
  out->warp_size = p.warpSize; out->max_threads_per_block = p.maxThreadsPerBlock;
  out->l2_bytes = p.l2CacheSize; out->max_shared_per_block_optin = (int)p.sharedMemPerBlockOptin;
  out->total_memory = p.totalGlobalMem;
  cudaDeviceGetAttribute(&out->clock_khz, cudaDevAttrClockRate, device);
  cudaDeviceGetAttribute(&out->memory_clock_khz, cudaDevAttrMemoryClockRate, device);
  return GFRT_OK;
}

GF_API int gfrt_memory_info(int device, unsigned long long* free_b, unsigned long long* total_b) {
  int prev = 0;
  cudaGetDevice(&prev);
  cudaError_t e = cudaSetDevice(device);
  if (e != cudaSuccess) return map_error(e);
  size_t f = 0, t = 0;
  e = cudaMemGetInfo(&f, &t);
  cudaSetDevice(prev);
  *free_b = f; *total_b = t;
  return map_error(e);
}

GF_API int gfrt_synchronize(int device) {
  int prev = 0;
  cudaGetDevice(&prev);
  cudaError_t e = cudaSetDevice(device);
  if (e != cudaSuccess) return map_error(e);
  e = cudaDeviceSynchronize();
  cudaSetDevice(prev);
  return map_error(e);
}

// ---- streams and events
GF_API int gfrt_stream_create(int device, int high_priority, void** out) {
  cudaError_t e = cudaSetDevice(device);
  if (e != cudaSuccess) return map_error(e);
  int lo = 0, hi = 0;
  cudaDeviceGetStreamPriorityRange(&lo, &hi);
  cudaStream_t s;
  e = cudaStreamCreateWithPriority(&s, cudaStreamNonBlocking, high_priority ? hi : lo);
  *out = s;
  return map_error(e);
}
GF_API int gfrt_stream_destroy(void* s) { return map_error(cudaStreamDestroy((cudaStream_t)s)); }
GF_API int gfrt_stream_synchronize(void* s) { return map_error(cudaStreamSynchronize((cudaStream_t)s)); }
GF_API int gfrt_stream_query(void* s) { return map_error(cudaStreamQuery((cudaStream_t)s)); }
// Device-side wait: later work on `s` waits for the event; the host does not block.
GF_API int gfrt_stream_wait_event(void* s, void* ev) {
  return map_error(cudaStreamWaitEvent((cudaStream_t)s, (cudaEvent_t)ev, 0));
}
GF_API int gfrt_event_create(int timing, void** out) {
  cudaEvent_t e;
  cudaError_t r = cudaEventCreateWithFlags(&e, timing ? cudaEventDefault : cudaEventDisableTiming);
  *out = e;
  return map_error(r);
}
GF_API int gfrt_event_destroy(void* e) { return map_error(cudaEventDestroy((cudaEvent_t)e)); }
GF_API int gfrt_event_record(void* e, void* s) { return map_error(cudaEventRecord((cudaEvent_t)e, (cudaStream_t)s)); }
GF_API int gfrt_event_synchronize(void* e) { return map_error(cudaEventSynchronize((cudaEvent_t)e)); }
GF_API int gfrt_event_query(void* e) { return map_error(cudaEventQuery((cudaEvent_t)e)); }
GF_API int gfrt_event_elapsed_ms(void* a, void* b, float* ms) {
  return map_error(cudaEventElapsedTime(ms, (cudaEvent_t)a, (cudaEvent_t)b));
}

// ---- pooled allocator
GF_API int gfrt_pool_create(int device, void** out) {
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess || device < 0 || device >= n) return GFRT_INVALID_DEVICE;
  Pool* p = new Pool();
  p->device = device;
  *out = p;
  return GFRT_OK;
}

GF_API int gfrt_pool_alloc(void* pool, unsigned long long nbytes, void** out) {
  Pool* p = (Pool*)pool;
  const size_t cls = size_class((size_t)nbytes);
  std::lock_guard<std::mutex> g(p->mu);
  auto& fl = p->free_lists[cls];
  void* ptr = nullptr;
  if (!fl.empty()) {
    ptr = fl.back();
    fl.pop_back();
    p->cached -= cls;
    ++p->hits;
  } else {
    int prev = 0;
    cudaGetDevice(&prev);
    cudaSetDevice(p->device);
    cudaError_t e = cudaMalloc(&ptr, cls);
    cudaSetDevice(prev);
    if (e != cudaSuccess) {
      cudaGetLastError();
      return map_error(e);
    }
    ++p->misses;
  }
  p->live[ptr] = cls;
  p->current += cls;
  if (p->current > p->peak) p->peak = p->current;
  *out = ptr;
  return GFRT_OK;
}

GF_API int gfrt_pool_free(void* pool, void* ptr) {
  Pool* p = (Pool*)pool;
  std::lock_guard<std::mutex> g(p->mu);
  auto it = p->live.find(ptr);
  if (it == p->live.end()) return GFRT_INVALID_VALUE;
  p->free_lists[it->second].push_back(ptr);
  p->current -= it->second;
  p->cached += it->second;
  p->live.erase(it);
  return GFRT_OK;
}

// Returns cached blocks to the driver.
GF_API int gfrt_pool_trim(void* pool) {
  Pool* p = (Pool*)pool;
  std::lock_guard<std::mutex> g(p->mu);
  for (auto& kv : p->free_lists)
    for (void* b : kv.second) cudaFree(b);
  p->free_lists.clear();
  p->cached = 0;
  return GFRT_OK;
}

// stats[0..5] = current, peak, cached, hits, misses, live blocks
GF_API int gfrt_pool_stats(void* pool, unsigned long long* stats) {
  Pool* p = (Pool*)pool;
  std::lock_guard<std::mutex> g(p->mu);
  stats[0] = p->current; stats[1] = p->peak; stats[2] = p->cached; stats[3] = p->hits; stats[4] = p->misses;
  stats[5] = p->live.size();
  return GFRT_OK;
}

GF_API int gfrt_pool_destroy(void* pool) {
  Pool* p = (Pool*)pool;
  gfrt_pool_trim(pool);
  for (auto& kv : p->live) cudaFree(kv.first);
  delete p;
  return GFRT_OK;
}
