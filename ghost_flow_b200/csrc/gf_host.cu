// Host-side helpers: driver entry point lookup, tensor-map encoding, device facts,
// and a per-device status word that kernels write their bounded-wait error codes to.
#include "gf_host.h"
#include <stdlib.h>

#include <atomic>
#include <mutex>

namespace gf {

EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q);
    if (e == cudaSuccess && q == cudaDriverEntryPointSuccess) fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

int make_tmap_2d(CUtensorMap* out, const void* base, CUtensorMapDataType dt, int elem_size, uint64_t rows,
                 uint64_t cols, uint64_t row_stride_bytes, uint32_t box_rows, uint32_t box_cols,
                 CUtensorMapSwizzle swz) {
  enter();
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return GFH_TMAP;
  if ((reinterpret_cast<uintptr_t>(base) & 15) || (row_stride_bytes & 15)) return GFH_BAD_ARG;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {row_stride_bytes};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swz,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    fprintf(stderr, "[ghost_flow_b200] tensor map encode failed: %d (rows=%llu cols=%llu pitch=%llu box=%ux%u)\n",
            (int)r, (unsigned long long)rows, (unsigned long long)cols, (unsigned long long)row_stride_bytes,
            box_rows, box_cols);
    return GFH_TMAP;
  }
  return GFH_OK;
}

int make_tmap_3d(CUtensorMap* out, const void* base, CUtensorMapDataType dt, int elem_size, uint64_t d2,
                 uint64_t rows, uint64_t cols, uint64_t row_stride_bytes, uint64_t d2_stride_bytes,
                 uint32_t box_d2, uint32_t box_rows, uint32_t box_cols, CUtensorMapSwizzle swz) {
  enter();
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return GFH_TMAP;
  if ((reinterpret_cast<uintptr_t>(base) & 15) || (row_stride_bytes & 15) || (d2_stride_bytes & 15))
    return GFH_BAD_ARG;
  cuuint64_t dims[3] = {cols, rows, d2};
  cuuint64_t strides[2] = {row_stride_bytes, d2_stride_bytes};
  cuuint32_t box[3] = {box_cols, box_rows, box_d2};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(out, dt, 3, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swz,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    fprintf(stderr, "[ghost_flow_b200] 3-D tensor map encode failed: %d\n", (int)r);
    return GFH_TMAP;
  }
  return GFH_OK;
}

static std::atomic<int> g_device{-1};
static std::atomic<long long> g_launches{0};

void note_extra_launches(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

// Every exported launcher calls this first: it binds the calling thread to the process's device in
// this library's copy of the CUDA runtime (PyTorch keeps its own copy, with its own per-thread state).
void enter() {
  g_launches.fetch_add(1, std::memory_order_relaxed);
  thread_local int bound = -2;
  const int d = g_device.load(std::memory_order_relaxed);
  if (d < 0) {
    if (bound == -2) {
      cudaFree(0);
      bound = -1;
    }
    return;
  }
  if (bound != d) {
    cudaSetDevice(d);
    bound = d;
  }
}

int process_device() { return g_device.load(std::memory_order_relaxed); }

int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) dev = 0;
  if (cached[dev] == 0) {
    int n = 0;
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    cached[dev] = n > 0 ? n : 148;
  }
  return cached[dev];
}

int attention_head_group(int heads) {
  static int env = -1;
  if (env < 0) {
    const char* e = getenv("GF_ATT_GROUP");
    env = e ? atoi(e) : 0;
  }
  int g = env > 0 ? env : 8;
  if (g > heads) g = heads;
  if (g < 1) g = 1;
  return g;
}

static int* g_check_buffers[32] = {};
int* check_buffer() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 32) return nullptr;
  return g_check_buffers[dev];
}
void set_check_buffer(int device, int* p) {
  if (device >= 0 && device < 32) g_check_buffers[device] = p;
}
}  // namespace gf

// ------------------------------------------------------------------ C surface
GF_API void gf_set_device(int dev) { gf::g_device.store(dev); }

// Kernels launched by this library since load (every launcher counts its own kernels).
GF_API long long gf_launch_count() { return gf::g_launches.load(); }

GF_API int gf_sm_count() { return gf::sm_count(); }
// 1 when the library was compiled with -DGF_CHECKED (data-dependent indices are range-checked on the device).
GF_API int gf_checked_build() {
#ifdef GF_CHECKED
  return 1;
#else
  return 0;
#endif
}
// status: int32[8] on `device` (word 0 = error code, words 1..7 = the report of a checked build).
GF_API int gf_set_check_buffer(int device, int* status) {
  gf::set_check_buffer(device, status);
  return 0;
}

GF_API int gf_device_count() {
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess) return 0;
  return n;
}

GF_API const char* gf_last_cuda_error() { return cudaGetErrorString(cudaPeekAtLastError()); }

GF_API int gf_version() { return 100; }
