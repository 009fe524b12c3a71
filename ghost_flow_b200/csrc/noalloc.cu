// gf_rmsnorm_bwd_noalloc: RMSNorm backward whose weight-gradient scratch lives in a fixed device
// array of this module, for callers that cannot allocate (see gf_noalloc.h for who they are, the
// size limit and the sharing rules). Same math as rmsnorm_bwd_kernel in norm.cu.
#include "gf_noalloc.h"

#include <mutex>

#include "gf_host.h"
#include "gf_ptx.cuh"

namespace gf {
namespace {

constexpr int NA_THREADS = 256;
constexpr int NA_MAXV = 4;  // 16-byte vectors per thread held in registers: D <= 256 * 4 * 8 = 8192

// Partial sums of dw, one row per block. Part of the module image: every GPU that loads the library
// holds these 148 * 8192 * 4 bytes until the process exits. In host code this name is only a handle for
// cudaGetSymbolAddress; it is not a device address and must never be passed to a kernel as one.
static __device__ __align__(256) float g_noalloc_scratch[GF_NOALLOC_MAX_PARTS * GF_NOALLOC_MAX_D];

__device__ __forceinline__ float na_warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float na_block_sum(float v, float* red) {
  v = na_warp_sum(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  __syncthreads();
  if (l == 0) red[w] = v;
  __syncthreads();
  float t = (l < (blockDim.x >> 5)) ? red[l] : 0.f;
  return na_warp_sum(t);
}
__device__ __forceinline__ void na_load8(const __nv_bfloat16* p, float (&f)[8]) {
  uint4 u = *reinterpret_cast<const uint4*>(p);
  float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}
__device__ __forceinline__ void na_store8(__nv_bfloat16* p, const float (&f)[8]) {
  uint4 u;
  u.x = pack_bf16x2(f[0], f[1]); u.y = pack_bf16x2(f[2], f[3]);
  u.z = pack_bf16x2(f[4], f[5]); u.w = pack_bf16x2(f[6], f[7]);
  *reinterpret_cast<uint4*>(p) = u;
}

// dx = rstd * g - x * rstd^3 * mean(g * x) (+ dres), g = dy * w. Block b writes its partial of
// dw = sum_rows dy * x * rstd to scratch row b (every column it owns, so stale contents never survive).
__global__ void __launch_bounds__(NA_THREADS)
na_rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                      const __nv_bfloat16* __restrict__ dy, const float* __restrict__ rstd_in,
                      const __nv_bfloat16* __restrict__ dres, __nv_bfloat16* __restrict__ dx,
                      float* __restrict__ scratch, int T, int D) {
  __shared__ float red[32];
  const int nv = D >> 3;
  float dwacc[NA_MAXV][8], wv[NA_MAXV][8];
#pragma unroll
  for (int i = 0; i < NA_MAXV; ++i) {
    const int v = threadIdx.x + i * NA_THREADS;
#pragma unroll
    for (int j = 0; j < 8; ++j) dwacc[i][j] = 0.f;
    if (v < nv) na_load8(w + v * 8, wv[i]);
  }
  for (int row = blockIdx.x; row < T; row += gridDim.x) {
    const float rstd = rstd_in[row];
    float xv[NA_MAXV][8], gv[NA_MAXV][8];
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < NA_MAXV; ++i) {
      const int v = threadIdx.x + i * NA_THREADS;
      if (v < nv) {
        na_load8(x + (long long)row * D + v * 8, xv[i]);
        na_load8(dy + (long long)row * D + v * 8, gv[i]);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          dwacc[i][j] += gv[i][j] * xv[i][j] * rstd;
          gv[i][j] *= wv[i][j];
          dot += gv[i][j] * xv[i][j];
        }
      }
    }
    dot = na_block_sum(dot, red);
    const float c = dot * rstd * rstd * rstd / (float)D;
#pragma unroll
    for (int i = 0; i < NA_MAXV; ++i) {
      const int v = threadIdx.x + i * NA_THREADS;
      if (v < nv) {
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = rstd * gv[i][j] - c * xv[i][j];
        if (dres) {
          float rv[8];
          na_load8(dres + (long long)row * D + v * 8, rv);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] += rv[j];
        }
        na_store8(dx + (long long)row * D + v * 8, o);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < NA_MAXV; ++i) {
    const int v = threadIdx.x + i * NA_THREADS;
    if (v < nv) {
      float* dst = scratch + (long long)blockIdx.x * D + v * 8;
#pragma unroll
      for (int j = 0; j < 8; ++j) dst[j] = dwacc[i][j];
    }
  }
}

__global__ void na_fold_kernel(const float* __restrict__ scratch, __nv_bfloat16* __restrict__ dw, int nparts, int D,
                               int accumulate) {
  const int d = blockIdx.x * blockDim.x + threadIdx.x;
  if (d >= D) return;
  float s = 0.f;
  for (int p = 0; p < nparts; ++p) s += scratch[(long long)p * D + d];
  if (accumulate) s += __bfloat162float(dw[d]);
  dw[d] = __float2bfloat16(s);
}

// Device address of the scratch array, looked up once per device with that device current.
float* scratch_address(int* err) {
  static float* addr[64] = {nullptr};
  static std::mutex mu;
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
    *err = GFH_CUDA;
    return nullptr;
  }
  std::lock_guard<std::mutex> lock(mu);
  if (addr[dev] == nullptr) {
    float* p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_noalloc_scratch);
    if (e != cudaSuccess || p == nullptr) {
      fprintf(stderr, "[ghost_flow_b200] gf_rmsnorm_bwd_noalloc: cudaGetSymbolAddress failed on device %d: %s\n",
              dev, cudaGetErrorString(e));
      *err = GFH_CUDA;
      return nullptr;
    }
    addr[dev] = p;
  }
  *err = GFH_OK;
  return addr[dev];
}

}  // namespace
}  // namespace gf

extern "C" int gf_rmsnorm_bwd_noalloc(const void* x, const void* w, const void* dy, const float* rstd,
                                      const void* dres, void* dx, void* dw, int T, int D, int accumulate,
                                      void* stream) {
  using namespace gf;
  // Bind this thread to the process's device in this library's runtime (no allocation involved). A plain
  // C caller that never selected a device simply uses the runtime's current device.
  // Arguments first: a call that is refused must not touch the device state of the calling thread.
  if (T <= 0 || D <= 0 || (D % 8) != 0 || !x || !w || !dy || !rstd || !dx || !dw) return GFH_BAD_ARG;
  // The kernels move rows as 16-byte vectors; a pointer into the middle of a buffer that is not 16-byte aligned
  // would fault on the device instead of failing here. rstd is read as fp32, dw written as bf16.
  const uintptr_t vec = reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w) |
                        reinterpret_cast<uintptr_t>(dy) | reinterpret_cast<uintptr_t>(dres) |
                        reinterpret_cast<uintptr_t>(dx);
  if ((vec & 15) || (reinterpret_cast<uintptr_t>(rstd) & 3) || (reinterpret_cast<uintptr_t>(dw) & 1))
    return GFH_BAD_ARG;
  if (D > GF_NOALLOC_MAX_D) {
    fprintf(stderr,
            "[ghost_flow_b200] gf_rmsnorm_bwd_noalloc: D = %d exceeds the built-in scratch (max D = %d); "
            "use gf_rmsnorm_bwd with a caller-provided scratch buffer instead\n",
            D, GF_NOALLOC_MAX_D);
    return GFH_TOO_LARGE;
  }
  const int want = process_device();
  if (want >= 0 && cudaSetDevice(want) != cudaSuccess) return GFH_CUDA;
  int err = GFH_OK;
  float* scratch = scratch_address(&err);
  if (!scratch) return err;
  const int parts = T < GF_NOALLOC_MAX_PARTS ? T : GF_NOALLOC_MAX_PARTS;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  na_rmsnorm_bwd_kernel<<<parts, NA_THREADS, 0, s>>>(
      reinterpret_cast<const __nv_bfloat16*>(x), reinterpret_cast<const __nv_bfloat16*>(w),
      reinterpret_cast<const __nv_bfloat16*>(dy), rstd, reinterpret_cast<const __nv_bfloat16*>(dres),
      reinterpret_cast<__nv_bfloat16*>(dx), scratch, T, D);
  na_fold_kernel<<<(D + 255) / 256, 256, 0, s>>>(scratch, reinterpret_cast<__nv_bfloat16*>(dw), parts, D, accumulate);
  note_extra_launches(2);
  return cudaGetLastError() == cudaSuccess ? GFH_OK : GFH_CUDA;
}
