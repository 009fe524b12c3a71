// Host-side helpers shared by the launchers: tensor-map encoding through the
// driver entry point (no link-time dependency on libcuda), status word access,
// and the C error codes of the library.
#pragma once
#include <atomic>
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#define GF_API extern "C" __attribute__((visibility("default")))

namespace gf {

enum HostErr : int {
  GFH_OK = 0,
  GFH_BAD_ARG = -1,
  GFH_CUDA = -2,
  GFH_TMAP = -3,
  GFH_TOO_LARGE = -4,
};

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn();

// Encode a 2-D tiled map over a row-major [rows, cols] view with `row_stride_bytes` pitch.
// Box = box_cols x box_rows elements, 128-byte swizzle (box_cols * elem_size must be 128 or less).
int make_tmap_2d(CUtensorMap* out, const void* base, CUtensorMapDataType dt, int elem_size, uint64_t rows,
                 uint64_t cols, uint64_t row_stride_bytes, uint32_t box_rows, uint32_t box_cols,
                 CUtensorMapSwizzle swz = CU_TENSOR_MAP_SWIZZLE_128B);

// 3-D map: [d2, rows, cols] with byte strides for rows and d2.
int make_tmap_3d(CUtensorMap* out, const void* base, CUtensorMapDataType dt, int elem_size, uint64_t d2,
                 uint64_t rows, uint64_t cols, uint64_t row_stride_bytes, uint64_t d2_stride_bytes,
                 uint32_t box_d2, uint32_t box_rows, uint32_t box_cols,
                 CUtensorMapSwizzle swz = CU_TENSOR_MAP_SWIZZLE_128B);

int sm_count();

// "The attributes of this kernel are set" per device. cudaFuncSetAttribute applies to the current device only, so a
// process that drives several GPUs has to repeat it on each; a single function-local bool would skip it on the
// second device. Races are benign (two threads may both set the same attribute to the same value).
struct DeviceOnce {
  std::atomic<unsigned char> done[64];
  DeviceOnce() { for (auto& d : done) d.store(0); }
  static int device() {
    int d = 0;
    if (cudaGetDevice(&d) != cudaSuccess || d < 0 || d >= 64) d = 0;
    return d;
  }
  bool todo() { return done[device()].load(std::memory_order_acquire) == 0; }
  void mark() { done[device()].store(1, std::memory_order_release); }
};
// The same for attributes that only ever grow (dynamic shared-memory limit raised to the largest request so far).
struct DeviceMax {
  std::atomic<size_t> value[64];
  DeviceMax() { for (auto& v : value) v.store(0); }
  size_t get() { return value[DeviceOnce::device()].load(std::memory_order_acquire); }
  void set(size_t v) { value[DeviceOnce::device()].store(v, std::memory_order_release); }
};
// Checked build: the 8-int status buffer of the current device (registered with gf_set_check_buffer), for kernels
// whose exported signature has no status pointer. Null when none was registered.
int* check_buffer();
void set_check_buffer(int device, int* p);

// Heads per dispatch group of the attention kernels: GF_ATT_GROUP when set (tuning), else 8, clamped to [1, heads].
int attention_head_group(int heads);

// Binds the calling thread to the device selected with gf_set_device (see gf_host.cu).
void enter();
// Launchers that start more than one kernel report the extra ones here (enter() counts one).
void note_extra_launches(int n);
// Device index selected with gf_set_device, or -1 when none was selected.
int process_device();

// Asks for the largest shared-memory carve-out for a kernel that itself needs little shared memory. An SM
// cannot change its L1/shared split while CTAs are resident, so a side-stream kernel running with the
// default split keeps the big-shared-memory GEMM / attention CTAs of the compute stream off every SM it
// occupies until it drains; with the same split they share the SM.
template <typename K>
inline void prefer_max_smem(K kernel) {
  cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
}

}  // namespace gf
