// fp8 (e4m3) quantisation kernels and the scaled fp8 GEMM on tcgen05 (kind::f8f6f4).
//
// The reference only emulates fp8 by rounding fp32 values (ghostflow-nn/src/mixed_precision.rs:264-285); here the
// operands are real e4m3 bytes and the product runs on the tensor cores at twice the bf16 rate.
//
// Two scaling schemes:
//   mode 0  one scale per row of A (token) and per row of B (output channel); the accumulator is scaled once in the
//           epilogue: C[m, n] = sa[m] * sb[n] * sum_k A[m, k] B[n, k].                      (128 x 256 tiles)
//   mode 1  block scales: A has one scale per row and 128-wide k block (stored [K / 128, M]), B one per 128 x 128
//           block ([N / 128, K / 128]). Every k block is accumulated in TMEM on its own and promoted into fp32
//           registers with its scale: C[m, n] = sum_kb sa[kb, m] * sb[n / 128, kb] * partial_kb.  (128 x 128 tiles)
//
// Layout of the kernel is the bf16 GEMM's: one TMA warp, one MMA warp, four epilogue warps, persistent over tiles,
// two TMEM accumulator buffers, bounded waits that record a status code and bail out.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>

#include "gf_host.h"
#include "gf_ptx.cuh"

namespace gf {

constexpr int F8_BM = 128;
constexpr int F8_BK = 128;          // e4m3 elements = 128 bytes = one swizzle-128B row
constexpr int F8_THREADS = 192;
constexpr float F8_MAX = 448.f;

// ------------------------------------------------------------------ quantisation
__device__ __forceinline__ uint32_t pack_e4m3x4(float a, float b, float c, float d) {
  const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
  const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
  return lo | (hi << 16);
}

// One warp per row. mode 0: scale[row]; mode 1: scale_t[kb * T + row] per 128-wide block.
__global__ void quant_rows_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, uint8_t* __restrict__ q,
                                  long long ldq, float* __restrict__ scale, int T, int K, int mode) {
  const int row = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (row >= T) return;
  const __nv_bfloat16* xr = x + (long long)row * ldx;
  uint8_t* qr = q + (long long)row * ldq;
  if (mode == 0) {
    float amax = 0.f;
    for (int c = lane * 8; c < K; c += 256) {
      const uint4 u = *reinterpret_cast<const uint4*>(xr + c);
      float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), cc = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
      amax = fmaxf(amax, fmaxf(fmaxf(fabsf(a.x), fabsf(a.y)), fmaxf(fabsf(b.x), fabsf(b.y))));
      amax = fmaxf(amax, fmaxf(fmaxf(fabsf(cc.x), fabsf(cc.y)), fmaxf(fabsf(d.x), fabsf(d.y))));
    }
    for (int o = 16; o; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const float s = fmaxf(amax, 1e-12f) / F8_MAX;
    const float inv = 1.f / s;
    if (lane == 0) scale[row] = s;
    for (int c = lane * 8; c < K; c += 256) {
      const uint4 u = *reinterpret_cast<const uint4*>(xr + c);
      float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), cc = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
      uint2 o;
      o.x = pack_e4m3x4(a.x * inv, a.y * inv, b.x * inv, b.y * inv);
      o.y = pack_e4m3x4(cc.x * inv, cc.y * inv, d.x * inv, d.y * inv);
      *reinterpret_cast<uint2*>(qr + c) = o;
    }
  } else {
    // 16 lanes cover one 128-wide block; a warp does two blocks per step
    for (int c0 = 0; c0 < K; c0 += 256) {
      const int c = c0 + lane * 8;
      float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      if (c < K) {
        const uint4 u = *reinterpret_cast<const uint4*>(xr + c);
        float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), cc = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
        v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y; v[4] = cc.x; v[5] = cc.y; v[6] = d.x; v[7] = d.y;
      }
      float amax = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(v[j]));
      for (int o = 8; o; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
      const float s = fmaxf(amax, 1e-12f) / F8_MAX;
      const float inv = 1.f / s;
      if (c < K) {
        if ((lane & 15) == 0) scale[(long long)(c >> 7) * T + row] = s;
        uint2 o;
        o.x = pack_e4m3x4(v[0] * inv, v[1] * inv, v[2] * inv, v[3] * inv);
        o.y = pack_e4m3x4(v[4] * inv, v[5] * inv, v[6] * inv, v[7] * inv);
        *reinterpret_cast<uint2*>(qr + c) = o;
      }
    }
  }
}

// One CTA (256 threads) per 128 x 128 block of a weight [N, K]; scale [N / 128 (ceil), K / 128].
__global__ void quant_block128_kernel(const __nv_bfloat16* __restrict__ w, long long ldw, uint8_t* __restrict__ q,
                                      long long ldq, float* __restrict__ scale, int N, int K) {
  __shared__ float red[8];
  const int kb = blockIdx.x, nb = blockIdx.y;
  const int c = kb * 128 + (threadIdx.x & 15) * 8;
  const int r0 = nb * 128 + (threadIdx.x >> 4);
  float amax = 0.f;
  for (int r = r0; r < min(N, nb * 128 + 128); r += 16) {
    if (c < K) {
      const uint4 u = *reinterpret_cast<const uint4*>(w + (long long)r * ldw + c);
      float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), cc = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
      amax = fmaxf(amax, fmaxf(fmaxf(fabsf(a.x), fabsf(a.y)), fmaxf(fabsf(b.x), fabsf(b.y))));
      amax = fmaxf(amax, fmaxf(fmaxf(fabsf(cc.x), fabsf(cc.y)), fmaxf(fabsf(d.x), fabsf(d.y))));
    }
  }
  for (int o = 16; o; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
  __syncthreads();
  amax = 0.f;
  for (int i = 0; i < 8; ++i) amax = fmaxf(amax, red[i]);
  const float s = fmaxf(amax, 1e-12f) / F8_MAX;
  const float inv = 1.f / s;
  if (threadIdx.x == 0) scale[(long long)nb * gridDim.x + kb] = s;
  for (int r = r0; r < min(N, nb * 128 + 128); r += 16) {
    if (c < K) {
      const uint4 u = *reinterpret_cast<const uint4*>(w + (long long)r * ldw + c);
      float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), cc = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
      uint2 o;
      o.x = pack_e4m3x4(a.x * inv, a.y * inv, b.x * inv, b.y * inv);
      o.y = pack_e4m3x4(cc.x * inv, cc.y * inv, d.x * inv, d.y * inv);
      *reinterpret_cast<uint2*>(q + (long long)r * ldq + c) = o;
    }
  }
}

// ------------------------------------------------------------------ GEMM
struct F8Params {
  int M, N, K;
  __nv_bfloat16* C;
  long long ldc;
  const float* sa;          // mode 0: [M]; mode 1: [K / 128, M]
  const float* sb;          // mode 0: [N]; mode 1: [ceil(N / 128), K / 128]
  const __nv_bfloat16* bias;
  int tiles_m, tiles_n;
  int* status;
  // split-K (mode 0, skinny problems): tile index = (k slice, tile); raw partial sums are added into `ws` [M, N]
  // with vector reductions and a second kernel applies scales and bias.
  int split_k;
  float* ws;
};

// Work item -> tile and k-block range. Returns false when the slice is empty.
__device__ __forceinline__ bool f8_item(const F8Params& p, int item, int num_kb, int& tm, int& tn, int& kb0, int& nkb) {
  const int per = p.tiles_m * p.tiles_n;
  const int ks = item / per;
  const int t = item - ks * per;
  tm = t % p.tiles_m;
  tn = t / p.tiles_m;
  const int kbs = (num_kb + p.split_k - 1) / p.split_k;
  kb0 = ks * kbs;
  nkb = min(kbs, num_kb - kb0);
  return nkb > 0;
}

template <int BN>
struct F8Cfg {
  static constexpr int A_BYTES = F8_BM * F8_BK;
  static constexpr int B_BYTES = BN * F8_BK;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = (BN == 256) ? 4 : 6;
  static constexpr int TMEM_COLS = 2 * BN;     // 512 or 256
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;
};

__device__ __forceinline__ void f8_set_status(int* status, int code) {
  if (status) atomicCAS(status, 0, code);
}

// MODE 0: BN = 256, one drain per tile. MODE 1: BN = 128, one drain per k block.
template <int BN, int MODE>
__global__ void __launch_bounds__(F8_THREADS, 1)
gemm_fp8_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const F8Params p) {
  using Cfg = F8Cfg<BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + Cfg::STAGES * Cfg::STAGE_BYTES);
  uint64_t* empty_bar = full_bar + Cfg::STAGES;
  uint64_t* tfull_bar = empty_bar + Cfg::STAGES;
  uint64_t* tempty_bar = tfull_bar + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_kb = (p.K + F8_BK - 1) / F8_BK;
  const int num_tiles = p.tiles_m * p.tiles_n * p.split_k;
  const int cta = blockIdx.x, nctas = gridDim.x;
  // accumulator hand-offs per tile: one (mode 0) or one per k block (mode 1)
  const int drains = MODE == 0 ? 1 : num_kb;

  if (threadIdx.x == 0) {
    for (int s = 0; s < Cfg::STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tfull_bar[b], 1);
      mbar_init(&tempty_bar[b], 4);
    }
    mbar_fence_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = cta; tile < num_tiles && ok; tile += nctas) {
        int tm, tn, kb0, nkb;
        if (!f8_item(p, tile, num_kb, tm, tn, kb0, nkb)) continue;
        for (int kb = kb0; kb < kb0 + nkb; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1)) {
            f8_set_status(p.status, GF_ERR_WAIT_EMPTY);
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * Cfg::STAGE_BYTES;
          mbar_expect_tx(&full_bar[stage], Cfg::STAGE_BYTES);
          tma_load_2d(sa, &tmA, &full_bar[stage], kb * F8_BK, tm * F8_BM);
          tma_load_2d(sa + Cfg::A_BYTES, &tmB, &full_bar[stage], kb * F8_BK, tn * BN);
          if (++stage == Cfg::STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_e4m3(F8_BM, BN);
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;      // accumulator hand-offs so far
      bool ok = true;
      for (int tile = cta; tile < num_tiles && ok; tile += nctas) {
        int tm_, tn_, kb0, nkb;
        if (!f8_item(p, tile, num_kb, tm_, tn_, kb0, nkb)) continue;
        for (int kb = kb0; kb < kb0 + nkb && ok; ++kb) {
          const bool first = MODE == 1 || kb == kb0;
          const int buf = it & 1;
          if (first) {
            if (!mbar_wait(&tempty_bar[buf], ((it >> 1) & 1) ^ 1)) {
              f8_set_status(p.status, GF_ERR_WAIT_TMEM_EMPTY);
              ok = false;
              break;
            }
            tc_fence_after();
          }
          if (!mbar_wait(&full_bar[stage], phase)) {
            f8_set_status(p.status, GF_ERR_WAIT_FULL);
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * Cfg::STAGE_BYTES);
          const uint32_t sb = sa + Cfg::A_BYTES;
          const uint32_t tmem_d = tmem_base + buf * BN;
#pragma unroll
          for (int kk = 0; kk < F8_BK / 32; ++kk) {
            const uint64_t adesc = umma_desc_sw128(sa + kk * 32, 16, 1024);
            const uint64_t bdesc = umma_desc_sw128(sb + kk * 32, 16, 1024);
            umma_f8_ss(tmem_d, adesc, bdesc, idesc, (kk > 0 || !first) ? 1u : 0u);
          }
          umma_commit(&empty_bar[stage]);
          if (++stage == Cfg::STAGES) {
            stage = 0;
            phase ^= 1;
          }
          if (MODE == 1 || kb == kb0 + nkb - 1) {
            umma_commit(&tfull_bar[buf]);
            ++it;
          }
        }
      }
    }
  } else {
    const int lane_grp = warp & 3;
    int it = 0;
    for (int tile = cta; tile < num_tiles; tile += nctas) {
      int tm, tn, kb0_, nkb_;
      if (!f8_item(p, tile, num_kb, tm, tn, kb0_, nkb_)) continue;
      const int row = tm * F8_BM + lane_grp * 32 + lane;
      const int n0 = tn * BN;
      bool ok = true;
      if constexpr (MODE == 0) {
        const int buf = it & 1;
        if (!mbar_wait_warp(&tfull_bar[buf], (it >> 1) & 1)) {
          f8_set_status(p.status, GF_ERR_WAIT_TMEM_FULL);
          break;
        }
        ++it;
        tc_fence_after();
        const float sa = row < p.M ? p.sa[row] : 0.f;
        const uint32_t taddr = tmem_base + buf * BN + ((uint32_t)(lane_grp * 32) << 16);
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t r[32];
          tmem_ld32(taddr + c * 32, r);
          tmem_ld_wait();
          const int col0 = n0 + c * 32;
          if (row < p.M && col0 < p.N && p.split_k > 1) {
            float* wp = p.ws + (long long)row * p.N + col0;
            if (col0 + 32 <= p.N && (p.N & 3) == 0) {
#pragma unroll
              for (int qd = 0; qd < 8; ++qd)
                asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(wp + qd * 4),
                             "f"(__uint_as_float(r[qd * 4])), "f"(__uint_as_float(r[qd * 4 + 1])),
                             "f"(__uint_as_float(r[qd * 4 + 2])), "f"(__uint_as_float(r[qd * 4 + 3])) : "memory");
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (col0 + j < p.N) atomicAdd(wp + j, __uint_as_float(r[j]));
            }
          } else if (row < p.M && col0 < p.N) {
            __nv_bfloat16* cp = p.C + (long long)row * p.ldc + col0;
            if (col0 + 32 <= p.N && (p.ldc & 7) == 0) {
#pragma unroll
              for (int qd = 0; qd < 4; ++qd) {
                float v[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                  v[j] = __uint_as_float(r[qd * 8 + j]) * sa * __ldg(p.sb + col0 + qd * 8 + j);
                  if (p.bias) v[j] += __bfloat162float(p.bias[col0 + qd * 8 + j]);
                }
                uint4 o;
                o.x = pack_bf16x2(v[0], v[1]); o.y = pack_bf16x2(v[2], v[3]);
                o.z = pack_bf16x2(v[4], v[5]); o.w = pack_bf16x2(v[6], v[7]);
                *reinterpret_cast<uint4*>(cp + qd * 8) = o;
              }
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (col0 + j < p.N) {
                  float v = __uint_as_float(r[j]) * sa * p.sb[col0 + j];
                  if (p.bias) v += __bfloat162float(p.bias[col0 + j]);
                  cp[j] = __float2bfloat16(v);
                }
            }
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tempty_bar[buf]);
      } else {
        float acc[BN];
#pragma unroll
        for (int j = 0; j < BN; ++j) acc[j] = 0.f;
        const uint32_t lane_addr = tmem_base + ((uint32_t)(lane_grp * 32) << 16);
        for (int kb = 0; kb < drains; ++kb) {
          const int buf = it & 1;
          if (!mbar_wait_warp(&tfull_bar[buf], (it >> 1) & 1)) {
            f8_set_status(p.status, GF_ERR_WAIT_TMEM_FULL);
            ok = false;
            break;
          }
          ++it;
          tc_fence_after();
          const float s = (row < p.M ? __ldg(p.sa + (long long)kb * p.M + row) : 0.f) *
                          __ldg(p.sb + (long long)tn * num_kb + kb);
#pragma unroll
          for (int c = 0; c < BN / 32; ++c) {
            uint32_t r[32];
            tmem_ld32(lane_addr + buf * BN + c * 32, r);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j) acc[c * 32 + j] = fmaf(s, __uint_as_float(r[j]), acc[c * 32 + j]);
          }
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&tempty_bar[buf]);
        }
        if (!ok) break;
        if (row < p.M) {
#pragma unroll
          for (int c = 0; c < BN / 8; ++c) {
            const int col = n0 + c * 8;
            if (col >= p.N) break;
            __nv_bfloat16* cp = p.C + (long long)row * p.ldc + col;
            if (col + 8 <= p.N && (p.ldc & 7) == 0) {
              float v[8];
#pragma unroll
              for (int j = 0; j < 8; ++j) v[j] = acc[c * 8 + j] + (p.bias ? __bfloat162float(p.bias[col + j]) : 0.f);
              uint4 o;
              o.x = pack_bf16x2(v[0], v[1]); o.y = pack_bf16x2(v[2], v[3]);
              o.z = pack_bf16x2(v[4], v[5]); o.w = pack_bf16x2(v[6], v[7]);
              *reinterpret_cast<uint4*>(cp) = o;
            } else {
#pragma unroll
              for (int j = 0; j < 8; ++j)
                if (col + j < p.N)
                  cp[j] = __float2bfloat16(acc[c * 8 + j] + (p.bias ? __bfloat162float(p.bias[col + j]) : 0.f));
            }
          }
        }
      }
    }
  }

  if (p.status && *reinterpret_cast<volatile int*>(p.status) != 0) error_drain_pause();
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
}

template <int BN, int MODE>
static int launch_f8(const CUtensorMap& tmA, const CUtensorMap& tmB, F8Params& p, cudaStream_t stream) {
  using Cfg = F8Cfg<BN>;
  static gf::DeviceOnce configured;
  auto kern = gemm_fp8_kernel<BN, MODE>;
  if (configured.todo()) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES) != cudaSuccess)
      return GFH_CUDA;
    configured.mark();
  }
  p.tiles_m = (p.M + F8_BM - 1) / F8_BM;
  p.tiles_n = (p.N + BN - 1) / BN;
  int grid = sm_count();
  if (p.tiles_m * p.tiles_n * p.split_k < grid) grid = p.tiles_m * p.tiles_n * p.split_k;
  kern<<<grid, F8_THREADS, Cfg::SMEM_BYTES, stream>>>(tmA, tmB, p);
  return cudaGetLastError() == cudaSuccess ? GFH_OK : GFH_CUDA;
}

__global__ void f8_splitk_finish_kernel(const float* __restrict__ ws, __nv_bfloat16* __restrict__ C, long long ldc,
                                        const float* __restrict__ sa, const float* __restrict__ sb,
                                        const __nv_bfloat16* __restrict__ bias, int M, int N) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long long)M * N) return;
  const int r = (int)(i / N), c = (int)(i % N);
  float v = ws[i] * sa[r] * sb[c];
  if (bias) v += __bfloat162float(bias[c]);
  C[(long long)r * ldc + c] = __float2bfloat16(v);
}

static float* g_f8_ws[32] = {};
static size_t g_f8_cap[32] = {};
static float* f8_workspace(size_t floats) {
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 32) return nullptr;
  if (g_f8_cap[dev] < floats) {
    if (g_f8_ws[dev]) cudaFree(g_f8_ws[dev]);
    size_t cap = floats < (size_t)(8 << 20) ? (size_t)(8 << 20) : floats;
    if (cudaMalloc(&g_f8_ws[dev], cap * sizeof(float)) != cudaSuccess) {
      g_f8_ws[dev] = nullptr;
      g_f8_cap[dev] = 0;
      cudaGetLastError();
      return nullptr;
    }
    g_f8_cap[dev] = cap;
  }
  return g_f8_ws[dev];
}

}  // namespace gf

using namespace gf;

// mode 0: scale [T]; mode 1: scale [K / 128, T] (K a multiple of 128).
GF_API int gf_quant_fp8_rows(const void* x, long long ldx, void* q, long long ldq, float* scale, int T, int K, int mode,
                             void* stream) {
  gf::enter();
  if (T <= 0 || K <= 0 || (K & 7) || (ldx & 7) || (ldq & 7) || (mode == 1 && (K & 127))) return GFH_BAD_ARG;
  const int wpb = 8;
  quant_rows_kernel<<<(T + wpb - 1) / wpb, wpb * 32, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)x, ldx, (uint8_t*)q, ldq, scale, T, K, mode);
  return cudaGetLastError() == cudaSuccess ? GFH_OK : GFH_CUDA;
}

// scale [ceil(N / 128), K / 128] (K a multiple of 128).
GF_API int gf_quant_fp8_block128(const void* w, long long ldw, void* q, long long ldq, float* scale, int N, int K,
                                 void* stream) {
  gf::enter();
  if (N <= 0 || K <= 0 || (K & 127) || (ldw & 7) || (ldq & 7)) return GFH_BAD_ARG;
  quant_block128_kernel<<<dim3(K / 128, (N + 127) / 128), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)w, ldw, (uint8_t*)q, ldq, scale, N, K);
  return cudaGetLastError() == cudaSuccess ? GFH_OK : GFH_CUDA;
}

// C[M, N] (bf16) = scaled A[M, K] (e4m3, K-major) x B[N, K]^T (e4m3, K-major); see the top of the file for `mode`.
GF_API int gf_gemm_fp8(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb,
                       long long ldc, const float* sa, const float* sb, const void* bias, int mode, int* status,
                       void* stream_v) {
  gf::enter();
  if (M <= 0 || N <= 0 || K <= 0 || (K & 15) || (lda & 15) || (ldb & 15) || !sa || !sb) return GFH_BAD_ARG;
  if (mode == 1 && (K & 127)) return GFH_BAD_ARG;
  const int bn = mode == 0 ? 256 : 128;
  CUtensorMap tmA, tmB;
  int rc = make_tmap_2d(&tmA, A, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, M, K, lda, F8_BM, F8_BK);
  if (rc) return rc;
  rc = make_tmap_2d(&tmB, B, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, N, K, ldb, bn, F8_BK);
  if (rc) return rc;
  F8Params p;
  p.M = M; p.N = N; p.K = K; p.C = (__nv_bfloat16*)C; p.ldc = ldc; p.sa = sa; p.sb = sb;
  p.bias = (const __nv_bfloat16*)bias; p.status = status;
  p.split_k = 1; p.ws = nullptr;
  cudaStream_t st = (cudaStream_t)stream_v;
  if (mode == 0 && M <= 256 && K >= 4096) {
    // decode-sized: split K until there is about one work item per SM (see the bf16 kernel)
    const long long tiles = (long long)((M + F8_BM - 1) / F8_BM) * ((N + 255) / 256);
    int split = (int)(sm_count() / (tiles > 0 ? tiles : 1));
    if (split > K / 1024) split = K / 1024;
    if (split > 16) split = 16;
    float* ws = split >= 2 ? f8_workspace((size_t)M * N) : nullptr;
    if (ws) {
      if (cudaMemsetAsync(ws, 0, sizeof(float) * (size_t)M * N, st) != cudaSuccess) return GFH_CUDA;
      p.split_k = split;
      p.ws = ws;
      rc = launch_f8<256, 0>(tmA, tmB, p, st);
      if (rc) return rc;
      const long long n = (long long)M * N;
      f8_splitk_finish_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(ws, (__nv_bfloat16*)C, ldc, sa, sb,
                                                                          (const __nv_bfloat16*)bias, M, N);
      gf::note_extra_launches(1);
      return cudaGetLastError() == cudaSuccess ? GFH_OK : GFH_CUDA;
    }
  }
  if (mode == 0) return launch_f8<256, 0>(tmA, tmB, p, st);
  if (mode == 1) return launch_f8<128, 1>(tmA, tmB, p, st);
  return GFH_BAD_ARG;
}
