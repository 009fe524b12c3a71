// bf16 GEMM on CTA pairs (tcgen05.mma.cta_group::2): two SMs of a cluster compute one 256 x 256 output tile.
//
//   C[M,N] = alpha * op(A)[M,K] * op(B)[K,N] (+ bias[N]) (+ residual[M,N]) (+ C when accumulating)
//
// Each CTA of a pair loads 128 rows of A and 128 of the 256 columns of B per 64-deep k block (32 KB instead of
// the 48 KB that a single CTA needs for a 128 x 256 tile), so the same shared memory holds seven stages instead of
// four and every byte that arrives from L2 feeds twice as many multiply-adds. The MMA is issued by one thread of
// the even CTA; it reads both CTAs' shared memory and writes 128 accumulator rows into each CTA's tensor memory.
// Protocol between the two CTAs (no multicast loads anywhere):
//   * TMA loads of both CTAs complete on the EVEN CTA's "full" barrier (cp.async.bulk.tensor ... .cta_group::2 with
//     the barrier address mapped into the even CTA); its producer thread posts the expected byte count of both.
//   * "stage empty" and "accumulator full" are tcgen05.commit arrivals, one to the local barrier and one to the
//     peer's (address mapped with mapa).
//   * "accumulator drained" is an mbarrier.arrive of the eight epilogue warps of both CTAs on the even CTA's barrier.
//   * cluster barriers at start (barriers initialised, TMEM allocated) and before exit (no signal may reach a CTA
//     that has gone).
// Every wait is bounded; a wait that runs out records a code in the status word and the role leaves its loop.
//
// Plain GEMMs only (all four operand layouts, the epilogue options of the single-CTA kernel); the fused roles
// (all-gather, reduce-scatter, grouped, split-K, implicit convolution) stay in gemm_bf16.cu.
// Replaces, like that file, ghostflow-cuda/src/optimized_kernels.cu:22-119 and ghostflow-cuda/src/blas.rs:278-313.
#include "gf_host.h"
#include "gf_ptx.cuh"
#include <stdlib.h>

namespace gf {

struct Gemm2Params {
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
  int tiles_m, tiles_n;     // 256 x BN tiles
  int band;                 // rows of tiles walked together (keeps one wave's A and B panels in L2)
  int act;                  // 0 none, 1 ReLU
};

constexpr int G2_BM = 128;        // rows of A per CTA
constexpr int G2_BK = 64;
constexpr int G2_THREADS = 192;   // TMA warp, MMA warp, 4 epilogue warps
constexpr int G2_A_BYTES = G2_BM * G2_BK * 2;

// BNH = rows of B (output columns) per CTA: 128 (256 x 256 tiles, seven stages) or 64 (256 x 128 tiles, nine
// stages; twice as many tiles, for problems whose last wave of 256-wide tiles would leave most pairs idle).
template <int BNH>
struct G2Cfg {
  static constexpr int BN = 2 * BNH;
  static constexpr int B_BYTES = BNH * G2_BK * 2;
  static constexpr int STAGE_BYTES = G2_A_BYTES + B_BYTES;
  static constexpr int STAGES = (BNH == 128) ? 7 : 9;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;
  static constexpr int TMEM_COLS = 2 * BN;      // two accumulator buffers
};

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// Address of the same shared-memory location in CTA `rank` of the cluster (shared::cluster window).
__device__ __forceinline__ uint32_t mapa_u32(uint32_t local_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire;" ::: "memory");
}
__device__ __forceinline__ void tmem_alloc_2sm(uint32_t* smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_2sm() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_2sm(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// 2-D tile load whose completion is signalled on a barrier given as a shared::cluster address (the even CTA's).
__device__ __forceinline__ void tma_load_2d_2sm(void* smem_dst, const CUtensorMap* m, uint32_t bar_cluster_addr, int x,
                                                int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar_cluster_addr), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void umma_bf16_ss_2sm(bool leader, uint32_t tmem_d, uint64_t adesc, uint64_t bdesc,
                                                 uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "setp.ne.b32 q, %5, 0;\n\t"
      "@q tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}\n"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"((uint32_t)leader)
      : "memory");
}
// Arrive on the barrier at a shared::cluster address once all MMAs issued so far by this thread have completed.
__device__ __forceinline__ void umma_commit_2sm(bool leader, uint32_t bar_cluster_addr) {
  asm volatile(
      "{\n\t.reg .pred q;\n\t"
      "setp.ne.b32 q, %1, 0;\n\t"
      "@q tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t}\n"
      ::"r"(bar_cluster_addr), "r"((uint32_t)leader)
      : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar_cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster_addr) : "memory");
}

__device__ __forceinline__ void g2_tile_coords(const Gemm2Params& p, int tile, int& tm, int& tn) {
  // bands of `band` tile rows; inside a band the row index runs fastest
  const int per_band = p.band * p.tiles_n;
  const int b = tile / per_band;
  const int first = b * p.band;
  const int rows = min(p.band, p.tiles_m - first);
  const int r = tile - b * per_band;
  tm = first + r % rows;
  tn = r / rows;
}

template <int BNH, bool A_MN, bool B_MN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(G2_THREADS, 1)
gemm2sm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    const Gemm2Params p) {
  using Cfg = G2Cfg<BNH>;
  constexpr int G2_BNH = BNH;
  constexpr int G2_BN = Cfg::BN;
  constexpr int G2_STAGES = Cfg::STAGES;
  constexpr int G2_STAGE_BYTES = Cfg::STAGE_BYTES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + G2_STAGES * G2_STAGE_BYTES);
  uint64_t* empty_bar = full_bar + G2_STAGES;
  uint64_t* tfull_bar = empty_bar + G2_STAGES;
  uint64_t* tempty_bar = tfull_bar + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const int num_kb = (p.K + G2_BK - 1) / G2_BK;
  const int num_tiles = p.tiles_m * p.tiles_n;
  const int pair = (int)blockIdx.x >> 1;
  const int npairs = (int)gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < G2_STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tfull_bar[b], 1);
      mbar_init(&tempty_bar[b], 8);     // four epilogue warps of each CTA (used in the even CTA)
    }
    mbar_fence_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tmem_alloc_2sm(tmem_slot, Cfg::TMEM_COLS);
    tmem_relinquish_2sm();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (one thread in each CTA)
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += npairs) {
        int tm, tn;
        g2_tile_coords(p, tile, tm, tn);
        const int m0 = tm * 2 * G2_BM + (int)rank * G2_BM;
        const int n0 = tn * G2_BN + (int)rank * G2_BNH;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1)) {
            if (p.status) atomicCAS(p.status, 0, GF_ERR_WAIT_EMPTY);
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * G2_STAGE_BYTES;
          uint8_t* sb = sa + G2_A_BYTES;
          if (rank == 0) mbar_expect_tx(&full_bar[stage], 2 * G2_STAGE_BYTES);   // both CTAs' bytes
          const uint32_t fb = mapa_u32(smem_u32(&full_bar[stage]), 0);
          const int k0 = kb * G2_BK;
          if (!A_MN) {
            tma_load_2d_2sm(sa, &tmA, fb, k0, m0);
          } else {
#pragma unroll
            for (int c = 0; c < G2_BM / 64; ++c) tma_load_2d_2sm(sa + c * (G2_BK * 128), &tmA, fb, m0 + c * 64, k0);
          }
          if (!B_MN) {
            tma_load_2d_2sm(sb, &tmB, fb, k0, n0);
          } else {
#pragma unroll
            for (int c = 0; c < G2_BNH / 64; ++c) tma_load_2d_2sm(sb + c * (G2_BK * 128), &tmB, fb, n0 + c * 64, k0);
          }
          if (++stage == G2_STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (even CTA only; uniform warp, one lane issues)
    if (rank == 0) {
      const bool leader = elect_one();
      constexpr uint32_t idesc = umma_idesc_bf16(2 * G2_BM, G2_BN, A_MN ? 1 : 0, B_MN ? 1 : 0);
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += npairs) {
        const int buf = it & 1;
        const uint32_t bphase = (it >> 1) & 1;
        ++it;
        if (!mbar_wait_warp(&tempty_bar[buf], bphase ^ 1)) {
          if (p.status && leader) atomicCAS(p.status, 0, GF_ERR_WAIT_TMEM_EMPTY);
          break;
        }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + buf * G2_BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait_warp(&full_bar[stage], phase)) {
            if (p.status && leader) atomicCAS(p.status, 0, GF_ERR_WAIT_FULL);
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * G2_STAGE_BYTES);
          const uint32_t sb = sa + G2_A_BYTES;
#pragma unroll
          for (int kk = 0; kk < G2_BK / 16; ++kk) {
            const uint64_t adesc = A_MN ? umma_desc_sw128(sa + kk * 2048, G2_BK * 128, 1024)
                                        : umma_desc_sw128(sa + kk * 32, 16, 1024);
            const uint64_t bdesc = B_MN ? umma_desc_sw128(sb + kk * 2048, G2_BK * 128, 1024)
                                        : umma_desc_sw128(sb + kk * 32, 16, 1024);
            umma_bf16_ss_2sm(leader, tmem_d, adesc, bdesc, idesc, (kb > 0 || kk > 0) ? 1u : 0u);
          }
          // the stage is free in both CTAs once these MMAs have read it
          const uint32_t eb = smem_u32(&empty_bar[stage]);
          umma_commit_2sm(leader, mapa_u32(eb, 0));
          umma_commit_2sm(leader, mapa_u32(eb, 1));
          if (++stage == G2_STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (ok) {
          const uint32_t tb = smem_u32(&tfull_bar[buf]);
          umma_commit_2sm(leader, mapa_u32(tb, 0));
          umma_commit_2sm(leader, mapa_u32(tb, 1));
        }
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5 of both CTAs)
    const int lane_grp = warp & 3;  // TMEM lanes [32*lane_grp, +32) belong to this warp
    int it = 0;
    for (int tile = pair; tile < num_tiles; tile += npairs) {
      int tm, tn;
      g2_tile_coords(p, tile, tm, tn);
      const int row = tm * 2 * G2_BM + (int)rank * G2_BM + lane_grp * 32 + lane;
      const int n0 = tn * G2_BN;
      const int buf = it & 1;
      const uint32_t bphase = (it >> 1) & 1;
      ++it;
      if (!mbar_wait_warp(&tfull_bar[buf], bphase)) {
        if (p.status) atomicCAS(p.status, 0, GF_ERR_WAIT_TMEM_FULL);
        break;
      }
      tc_fence_after();
      const uint32_t taddr = tmem_base + buf * G2_BN + ((uint32_t)(lane_grp * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < G2_BN / 32; ++c) {
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
          if (p.act == 1) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = fmaxf(v[j], 0.f);
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
      if (lane == 0) mbar_arrive_cluster(mapa_u32(smem_u32(&tempty_bar[buf]), 0));
    }
  }

  // ------------------------------------------------------------ teardown
  if (p.status && *reinterpret_cast<volatile int*>(p.status) != 0) error_drain_pause();
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();     // nothing of this pair is in flight any more: barriers and TMEM may go
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc_2sm(tmem_base, Cfg::TMEM_COLS);
  }
}

template <int BNH, bool A_MN, bool B_MN>
static int launch_gemm2(const CUtensorMap& tmA, const CUtensorMap& tmB, Gemm2Params& p, cudaStream_t stream) {
  using Cfg = G2Cfg<BNH>;
  constexpr int G2_SMEM_BYTES = Cfg::SMEM_BYTES;
  constexpr int G2_BN = Cfg::BN;
  static gf::DeviceOnce configured;
  static int max_pairs = 0;
  auto kern = gemm2sm_bf16_kernel<BNH, A_MN, B_MN>;
  if (configured.todo()) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, G2_SMEM_BYTES) != cudaSuccess)
      return GFH_CUDA;
    // how many CTA pairs the device can hold at once (a GPC with an odd number of free SMs strands one)
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(sm_count() & ~1);
    cfg.blockDim = dim3(G2_THREADS);
    cfg.dynamicSmemBytes = G2_SMEM_BYTES;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeClusterDimension;
    at[0].val.clusterDim.x = 2; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
    cfg.attrs = at; cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess || n <= 0) {
      cudaGetLastError();
      n = sm_count() / 2;
    }
    max_pairs = n;
    configured.mark();
  }
  p.tiles_m = (p.M + 2 * G2_BM - 1) / (2 * G2_BM);
  p.tiles_n = (p.N + G2_BN - 1) / G2_BN;
  const int tiles = p.tiles_m * p.tiles_n;
  int pairs = max_pairs < tiles ? max_pairs : tiles;
  if (pairs < 1) pairs = 1;
  p.band = p.tiles_m > 8 ? 8 : p.tiles_m;
  kern<<<2 * pairs, G2_THREADS, G2_SMEM_BYTES, stream>>>(tmA, tmB, p);
  return cudaGetLastError() == cudaSuccess ? GFH_OK : GFH_CUDA;
}

// 1 when plain GEMMs of this shape should run on CTA pairs. GF_GEMM_2SM=0 turns the path off, =1 forces it for
// every shape it can take.
int gemm2sm_wanted(int M, int N, int K) {
  static int mode = -1;
  if (mode < 0) {
    const char* e = getenv("GF_GEMM_2SM");
    mode = e ? atoi(e) : 2;
  }
  if (mode == 0) return 0;
  if (mode == 1) return 1;
  // default: problems with enough 256 x 256 tiles to give every pair work
  const long long tiles = (long long)((M + 255) / 256) * ((N + 255) / 256);
  return tiles >= (sm_count() / 2) && K >= 256;
}

// Width of the pair's tile for this problem. 256 x 128 tiles measure 1.28x slower per flop than 256 x 256 ones
// (8192^3: 0.898 vs 0.699 ms), more than a fuller last wave can win back on the shapes tried (4096^3: 0.116 vs
// 0.095 ms), so they are only used for narrow outputs. GF_GEMM_2SM_BN=128|256 forces one.
static int g2_pick_bn(int M, int N) {
  static int forced = -1;
  if (forced < 0) {
    const char* e = getenv("GF_GEMM_2SM_BN");
    forced = e ? atoi(e) : 0;
  }
  if (forced == 128 || forced == 256) return forced;
  (void)M;
  return N <= 128 ? 128 : 256;
}

int gemm2sm_run(const void* A, const void* B, void* C, int M, int N, int K, int a_mn_major, long long lda,
                int b_mn_major, long long ldb, long long ldc, int out_fp32, int accumulate, const void* bias,
                const void* residual, long long ldr, float alpha, int* status, int activation, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return GFH_BAD_ARG;
  const int bn = g2_pick_bn(M, N);
  CUtensorMap tmA, tmB;
  int rc;
  if (!a_mn_major) rc = make_tmap_2d(&tmA, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, M, K, lda * 2, G2_BM, G2_BK);
  else rc = make_tmap_2d(&tmA, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, M, lda * 2, G2_BK, 64);
  if (rc) return rc;
  if (!b_mn_major) rc = make_tmap_2d(&tmB, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, N, K, ldb * 2, bn / 2, G2_BK);
  else rc = make_tmap_2d(&tmB, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, N, ldb * 2, G2_BK, 64);
  if (rc) return rc;
  Gemm2Params p;
  p.M = M; p.N = N; p.K = K; p.C = C; p.ldc = ldc; p.out_fp32 = out_fp32; p.accumulate = accumulate;
  p.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  p.residual = reinterpret_cast<const __nv_bfloat16*>(residual);
  p.ldr = ldr; p.alpha = alpha; p.status = status; p.act = activation == 1 ? 1 : 0;
#define GF_G2_DISPATCH(BNH_)                                                                        \
  if (!a_mn_major && !b_mn_major) return launch_gemm2<BNH_, false, false>(tmA, tmB, p, stream);     \
  if (!a_mn_major && b_mn_major) return launch_gemm2<BNH_, false, true>(tmA, tmB, p, stream);       \
  if (a_mn_major && !b_mn_major) return launch_gemm2<BNH_, true, false>(tmA, tmB, p, stream);       \
  return launch_gemm2<BNH_, true, true>(tmA, tmB, p, stream);
  if (bn == 256) { GF_G2_DISPATCH(128) }
  GF_G2_DISPATCH(64)
#undef GF_G2_DISPATCH
}

}  // namespace gf
