// Persistent, warp-specialised bf16 GEMM for sm_100a.
//
//   C[M,N] = alpha * op(A)[M,K] * op(B)[K,N] (+ bias[N]) (+ residual[M,N]) (+ C when accumulating)
//
// Operands arrive by TMA into 128-byte-swizzled shared-memory stages, one elected
// thread issues tcgen05.mma (128 x BN x 16) into a double-buffered TMEM accumulator,
// and four epilogue warps drain TMEM with tcgen05.ld while the next tile's MMAs run.
// Each operand may be K-major (reduction index contiguous) or MN-major (row/column
// index contiguous), so forward, dgrad and wgrad GEMMs need no transposed copies.
//
// Replaces the reference's fp32 shared-memory SGEMM and its wmma kernel
// (ghostflow-cuda/src/optimized_kernels.cu:22-119) and the cuBLAS wrapper
// (ghostflow-cuda/src/blas.rs:278-313).
#include "gf_host.h"
#include "gf_ptx.cuh"

namespace gf {

struct GemmParams {
  int M, N, K;
  void* C;
  long long ldc;
  int out_fp32;
  int accumulate;
  const __nv_bfloat16* bias;
  const __nv_bfloat16* residual;
  long long ldr;
  float alpha;
  int* status;
  int tiles_m, tiles_n;
  // Optional readiness flags for operand B (used by the fused all-gather + GEMM path):
  // tile column block n waits until b_ready[n_to_flag(n)] >= b_epoch. Null = no waiting.
  const int* b_ready;
  int b_rows_per_flag;
  int b_epoch;
};

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int GEMM_THREADS = 192;

template <int BN>
struct GemmCfg {
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = (BN == 256) ? 4 : 6;
  static constexpr int TMEM_COLS = (2 * BN >= 512) ? 512 : (2 * BN >= 256 ? 256 : 128);
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;
};

__device__ __forceinline__ void set_status(int* status, int code) {
  if (status) atomicCAS(status, 0, code);
}

template <int BN, bool A_MN, bool B_MN>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const GemmParams p) {
  using Cfg = GemmCfg<BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + Cfg::STAGES * Cfg::STAGE_BYTES);
  uint64_t* empty_bar = full_bar + Cfg::STAGES;
  uint64_t* tfull_bar = empty_bar + Cfg::STAGES;
  uint64_t* tempty_bar = tfull_bar + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_kb = (p.K + BK - 1) / BK;
  const int num_tiles = p.tiles_m * p.tiles_n;

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
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const int tm = tile % p.tiles_m;
        const int tn = tile / p.tiles_m;
        const int m0 = tm * BM, n0 = tn * BN;
        if (p.b_ready) {
          // Wait (bounded) until every row block of B that this tile reads has landed in local memory.
          const int f0 = n0 / p.b_rows_per_flag;
          int n_hi = n0 + BN - 1;
          if (n_hi > p.N - 1) n_hi = p.N - 1;
          const int f1 = n_hi / p.b_rows_per_flag;
          for (int f = f0; f <= f1 && ok; ++f) {
            uint32_t it = 0;
            while (true) {
              int v;
              asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p.b_ready + f) : "memory");
              if (v >= p.b_epoch) break;
              if (++it > GF_WAIT_LIMIT) {
                ok = false;
                break;
              }
              __nanosleep(64);
            }
          }
          if (!ok) {
            set_status(p.status, GF_ERR_WAIT_PEER);
            break;
          }
          fence_proxy_async_all();
        }
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1)) {
            set_status(p.status, GF_ERR_WAIT_EMPTY);
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * Cfg::STAGE_BYTES;
          uint8_t* sb = sa + Cfg::A_BYTES;
          mbar_expect_tx(&full_bar[stage], Cfg::STAGE_BYTES);
          const int k0 = kb * BK;
          if (!A_MN) {
            tma_load_2d(sa, &tmA, &full_bar[stage], k0, m0);
          } else {
#pragma unroll
            for (int c = 0; c < BM / 64; ++c) tma_load_2d(sa + c * (BK * 128), &tmA, &full_bar[stage], m0 + c * 64, k0);
          }
          if (!B_MN) {
            tma_load_2d(sb, &tmB, &full_bar[stage], k0, n0);
          } else {
#pragma unroll
            for (int c = 0; c < BN / 64; ++c) tma_load_2d(sb + c * (BK * 128), &tmB, &full_bar[stage], n0 + c * 64, k0);
          }
          if (++stage == Cfg::STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_bf16(BM, BN, A_MN ? 1 : 0, B_MN ? 1 : 0);
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++it) {
        const int buf = it & 1;
        const uint32_t bphase = (it >> 1) & 1;
        if (!mbar_wait(&tempty_bar[buf], bphase ^ 1)) {
          set_status(p.status, GF_ERR_WAIT_TMEM_EMPTY);
          break;
        }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + buf * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase)) {
            set_status(p.status, GF_ERR_WAIT_FULL);
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * Cfg::STAGE_BYTES);
          const uint32_t sb = sa + Cfg::A_BYTES;
#pragma unroll
          for (int kk = 0; kk < BK / 16; ++kk) {
            const uint64_t adesc = A_MN ? umma_desc_sw128(sa + kk * 2048, BK * 128, 1024)
                                        : umma_desc_sw128(sa + kk * 32, 16, 1024);
            const uint64_t bdesc = B_MN ? umma_desc_sw128(sb + kk * 2048, BK * 128, 1024)
                                        : umma_desc_sw128(sb + kk * 32, 16, 1024);
            umma_bf16_ss(tmem_d, adesc, bdesc, idesc, (kb > 0 || kk > 0) ? 1u : 0u);
          }
          umma_commit(&empty_bar[stage]);
          if (++stage == Cfg::STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (ok) umma_commit(&tfull_bar[buf]);
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5)
    const int lane_grp = warp & 3;  // TMEM lanes [32*lane_grp, +32) belong to this warp
    int it = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++it) {
      const int buf = it & 1;
      const uint32_t bphase = (it >> 1) & 1;
      const int tm = tile % p.tiles_m;
      const int tn = tile / p.tiles_m;
      const int row = tm * BM + lane_grp * 32 + lane;
      const int n0 = tn * BN;
      if (!mbar_wait_warp(&tfull_bar[buf], bphase)) {
        set_status(p.status, GF_ERR_WAIT_TMEM_FULL);
        break;
      }
      tc_fence_after();
      const uint32_t taddr = tmem_base + buf * BN + ((uint32_t)(lane_grp * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld32(taddr + c * 32, r);
        tmem_ld_wait();
        const int col0 = n0 + c * 32;
        if (row < p.M && col0 < p.N) {
          float v[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]) * p.alpha;
          const bool full = (col0 + 32 <= p.N);
          if (p.bias) {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (full || col0 + j < p.N) v[j] += __bfloat162float(p.bias[col0 + j]);
          }
          if (p.residual) {
            const __nv_bfloat16* rp = p.residual + (long long)row * p.ldr + col0;
            if (full && ((p.ldr & 7) == 0)) {
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                uint4 u = *reinterpret_cast<const uint4*>(rp + q * 8);
                float2 f0 = unpack_bf16x2(u.x), f1 = unpack_bf16x2(u.y), f2 = unpack_bf16x2(u.z),
                       f3 = unpack_bf16x2(u.w);
                v[q * 8 + 0] += f0.x; v[q * 8 + 1] += f0.y; v[q * 8 + 2] += f1.x; v[q * 8 + 3] += f1.y;
                v[q * 8 + 4] += f2.x; v[q * 8 + 5] += f2.y; v[q * 8 + 6] += f3.x; v[q * 8 + 7] += f3.y;
              }
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (col0 + j < p.N) v[j] += __bfloat162float(rp[j]);
            }
          }
          if (p.out_fp32) {
            float* cp = reinterpret_cast<float*>(p.C) + (long long)row * p.ldc + col0;
            if (full && ((p.ldc & 3) == 0)) {
#pragma unroll
              for (int q = 0; q < 8; ++q) {
                float4 o = make_float4(v[q * 4], v[q * 4 + 1], v[q * 4 + 2], v[q * 4 + 3]);
                if (p.accumulate) {
                  float4 old = *reinterpret_cast<float4*>(cp + q * 4);
                  o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
                }
                *reinterpret_cast<float4*>(cp + q * 4) = o;
              }
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (col0 + j < p.N) cp[j] = p.accumulate ? cp[j] + v[j] : v[j];
            }
          } else {
            __nv_bfloat16* cp = reinterpret_cast<__nv_bfloat16*>(p.C) + (long long)row * p.ldc + col0;
            if (full && ((p.ldc & 7) == 0)) {
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                if (p.accumulate) {
                  uint4 u = *reinterpret_cast<uint4*>(cp + q * 8);
                  float2 f0 = unpack_bf16x2(u.x), f1 = unpack_bf16x2(u.y), f2 = unpack_bf16x2(u.z),
                         f3 = unpack_bf16x2(u.w);
                  v[q * 8 + 0] += f0.x; v[q * 8 + 1] += f0.y; v[q * 8 + 2] += f1.x; v[q * 8 + 3] += f1.y;
                  v[q * 8 + 4] += f2.x; v[q * 8 + 5] += f2.y; v[q * 8 + 6] += f3.x; v[q * 8 + 7] += f3.y;
                }
                uint4 o;
                o.x = pack_bf16x2(v[q * 8 + 0], v[q * 8 + 1]);
                o.y = pack_bf16x2(v[q * 8 + 2], v[q * 8 + 3]);
                o.z = pack_bf16x2(v[q * 8 + 4], v[q * 8 + 5]);
                o.w = pack_bf16x2(v[q * 8 + 6], v[q * 8 + 7]);
                *reinterpret_cast<uint4*>(cp + q * 8) = o;
              }
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (col0 + j < p.N) {
                  float o = v[j];
                  if (p.accumulate) o += __bfloat162float(cp[j]);
                  cp[j] = __float2bfloat16(o);
                }
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty_bar[buf]);
    }
  }

  // ------------------------------------------------------------ teardown
  if (p.status && *reinterpret_cast<volatile int*>(p.status) != 0) error_drain_pause();
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
}

template <int BN, bool A_MN, bool B_MN>
static int launch_gemm(const CUtensorMap& tmA, const CUtensorMap& tmB, GemmParams& p, int max_ctas,
                       cudaStream_t stream) {
  using Cfg = GemmCfg<BN>;
  static bool configured = false;
  auto kern = gemm_bf16_kernel<BN, A_MN, B_MN>;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES);
    if (e != cudaSuccess) return GFH_CUDA;
    configured = true;
  }
  p.tiles_m = (p.M + BM - 1) / BM;
  p.tiles_n = (p.N + BN - 1) / BN;
  int tiles = p.tiles_m * p.tiles_n;
  int grid = sm_count();
  if (max_ctas > 0 && max_ctas < grid) grid = max_ctas;
  if (tiles < grid) grid = tiles;
  kern<<<grid, GEMM_THREADS, Cfg::SMEM_BYTES, stream>>>(tmA, tmB, p);
  return cudaGetLastError() == cudaSuccess ? GFH_OK : GFH_CUDA;
}

static int pick_bn(int M, int N, int hint) {
  if (hint == 128 || hint == 256) return hint;
  const int sms = sm_count();
  auto eff = [&](int bn) {
    long long tiles = (long long)((M + BM - 1) / BM) * ((N + bn - 1) / bn);
    long long waves = (tiles + sms - 1) / sms;
    return (double)tiles / (double)(waves * sms);
  };
  if (N <= 128) return 128;
  // 256-wide tiles need a third fewer operand bytes per flop and measure about 1.35x faster per tile
  // than 128-wide ones (4096^3: 1266 vs 932 TFLOP/s), so 128 only pays when 256-wide tiles would leave
  // most of the machine idle (small problems).
  return (eff(128) > eff(256) * 1.45) ? 128 : 256;
}

}  // namespace gf

// lda/ldb: row pitch in elements of the matrix as stored.
//   a_mn_major = 0: A stored [M, K] (K contiguous); 1: A stored [K, M] (M contiguous).
//   b_mn_major = 0: B stored [N, K] (K contiguous); 1: B stored [K, N] (N contiguous).
GF_API int gf_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, int a_mn_major, long long lda,
                        int b_mn_major, long long ldb, long long ldc, int out_fp32, int accumulate,
                        const void* bias, const void* residual, long long ldr, float alpha, int* status,
                        int bn_hint, int max_ctas, const int* b_ready, int b_rows_per_flag, int b_epoch,
                        void* stream_v) {
  gf::enter();
  using namespace gf;
  if (M <= 0 || N <= 0 || K <= 0) return GFH_BAD_ARG;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_v);
  const int bn = pick_bn(M, N, bn_hint);
  CUtensorMap tmA, tmB;
  int rc;
  if (!a_mn_major)
    rc = make_tmap_2d(&tmA, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, M, K, lda * 2, BM, BK);
  else
    rc = make_tmap_2d(&tmA, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, M, lda * 2, BK, 64);
  if (rc) return rc;
  if (!b_mn_major)
    rc = make_tmap_2d(&tmB, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, N, K, ldb * 2, bn, BK);
  else
    rc = make_tmap_2d(&tmB, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, N, ldb * 2, BK, 64);
  if (rc) return rc;
  GemmParams p;
  p.M = M; p.N = N; p.K = K;
  p.C = C; p.ldc = ldc; p.out_fp32 = out_fp32; p.accumulate = accumulate;
  p.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  p.residual = reinterpret_cast<const __nv_bfloat16*>(residual);
  p.ldr = ldr; p.alpha = alpha; p.status = status;
  p.b_ready = b_ready; p.b_rows_per_flag = b_rows_per_flag > 0 ? b_rows_per_flag : 1; p.b_epoch = b_epoch;
#define GF_DISPATCH(BN_)                                                                  \
  if (!a_mn_major && !b_mn_major) return launch_gemm<BN_, false, false>(tmA, tmB, p, max_ctas, stream); \
  if (!a_mn_major && b_mn_major) return launch_gemm<BN_, false, true>(tmA, tmB, p, max_ctas, stream);   \
  if (a_mn_major && !b_mn_major) return launch_gemm<BN_, true, false>(tmA, tmB, p, max_ctas, stream);   \
  return launch_gemm<BN_, true, true>(tmA, tmB, p, max_ctas, stream);
  if (bn == 256) { GF_DISPATCH(256) }
  GF_DISPATCH(128)
#undef GF_DISPATCH
}
