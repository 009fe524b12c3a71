// FlashAttention forward, second generation: one CTA owns 256 query rows of one head as two
// 128-row tiles, each with its own four softmax warps, so the tensor core works on one tile
// (S = Q K^T or O += P V) while the other tile's warps run their softmax. The output accumulates
// in TMEM across KV tiles; it is rescaled in place (tcgen05.ld -> multiply -> tcgen05.st) only when a
// row maximum has grown by more than 2^8 since the last rescale, which after the first tiles is rare.
// P is exp2 of the raw scores against that (possibly stale) reference maximum, so it stays below 2^8.
//
// Tensor layouts and the math are those of attn_fwd.cu, which stays as the fallback for shapes this
// kernel does not take. Replaces ghostflow-cuda/src/optimized_kernels.cu:185-248 and the CPU algorithm of
// ghostflow-nn/src/flash_attention.rs:122-250.
#include "gf_host.h"
#include "gf_ptx.cuh"

namespace gf {

constexpr int F2_TILE = 128;      // query rows per tile, kv rows per step
constexpr int F2_THREADS = 320;   // TMA warp, MMA warp, 2 x 4 softmax warps
constexpr float F2_RESCALE_THRESHOLD = 8.0f;  // log2 units

struct Fa2Params {
  int B, S, Hq, Hkv;
  int causal;
  float scale;
  __nv_bfloat16* O;
  long long ldo;
  float* lse;
  int* status;
};

template <int HD>
struct Fa2Cfg {
  static constexpr int CH = HD / 64;
  static constexpr int TILE_BYTES = F2_TILE * HD * 2;      // one Q / K / V tile
  static constexpr int P_BYTES = F2_TILE * F2_TILE * 2;
  static constexpr int OFF_Q = 0;                           // 2 tiles
  static constexpr int OFF_K = OFF_Q + 2 * TILE_BYTES;      // 1 stage
  static constexpr int OFF_V = OFF_K + TILE_BYTES;          // 2 stages
  static constexpr int OFF_P = OFF_V + 2 * TILE_BYTES;      // 2 tiles
  static constexpr int OFF_BAR = OFF_P + 2 * P_BYTES;
  static constexpr int SMEM_BYTES = OFF_BAR + 256 + 1024;
  static constexpr int TM_S = 0;      // + t * 128
  static constexpr int TM_O = 256;    // + t * 128
  static constexpr int TMEM_COLS = 512;
};

template <int HD>
__global__ void __launch_bounds__(F2_THREADS, 1)
fa_fwd2_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
               const __grid_constant__ CUtensorMap tmV, const Fa2Params p) {
  using Cfg = Fa2Cfg<HD>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem + Cfg::OFF_Q;
  uint8_t* sK = smem + Cfg::OFF_K;
  uint8_t* sV = smem + Cfg::OFF_V;
  uint8_t* sP = smem + Cfg::OFF_P;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::OFF_BAR);
  uint64_t* q_full = bars + 0;
  uint64_t* k_full = bars + 1;
  uint64_t* k_empty = bars + 2;
  uint64_t* v_full = bars + 3;    // [2]
  uint64_t* v_empty = bars + 5;   // [2]
  uint64_t* s_full = bars + 7;    // [2] per tile
  uint64_t* s_empty = bars + 9;   // [2]
  uint64_t* p_full = bars + 11;   // [2]
  uint64_t* pv_done = bars + 13;  // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 15);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_qb = (p.S + 2 * F2_TILE - 1) / (2 * F2_TILE);
  const int qb = n_qb - 1 - (int)blockIdx.x;  // heaviest blocks first
  const int h = blockIdx.y, b = blockIdx.z;
  const int hk = h / (p.Hq / p.Hkv);
  const int n_kv_all = (p.S + F2_TILE - 1) / F2_TILE;
  const int row_base = b * p.S;
  int n_kv[2];
#pragma unroll
  for (int t = 0; t < 2; ++t) {
    const int q0 = qb * 2 * F2_TILE + t * F2_TILE;
    if (q0 >= p.S) n_kv[t] = 0;
    else n_kv[t] = p.causal ? min(q0 / F2_TILE + 1, n_kv_all) : n_kv_all;
  }
  const int n_j = max(n_kv[0], n_kv[1]);

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    mbar_init(k_full, 1);
    mbar_init(k_empty, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&s_empty[i], 4);
      mbar_init(&p_full[i], 4);
      mbar_init(&pv_done[i], 1);
    }
    mbar_fence_init();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
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
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      mbar_expect_tx(q_full, 2 * Cfg::TILE_BYTES);
#pragma unroll
      for (int t = 0; t < 2; ++t)
#pragma unroll
        for (int c = 0; c < Cfg::CH; ++c)
          tma_load_2d(sQ + t * Cfg::TILE_BYTES + c * (F2_TILE * 128), &tmQ, q_full, h * HD + c * 64,
                      row_base + qb * 2 * F2_TILE + t * F2_TILE);
      for (int j = 0; j < n_j; ++j) {
        if (!mbar_wait(k_empty, (j & 1) ^ 1)) {
          if (p.status) atomicCAS(p.status, 0, GF_ERR_WAIT_EMPTY);
          break;
        }
        mbar_expect_tx(k_full, Cfg::TILE_BYTES);
#pragma unroll
        for (int c = 0; c < Cfg::CH; ++c)
          tma_load_2d(sK + c * (F2_TILE * 128), &tmK, k_full, hk * HD + c * 64, row_base + j * F2_TILE);
        const int st = j & 1;
        if (!mbar_wait(&v_empty[st], ((j >> 1) & 1) ^ 1)) {
          if (p.status) atomicCAS(p.status, 0, GF_ERR_WAIT_EMPTY);
          break;
        }
        mbar_expect_tx(&v_full[st], Cfg::TILE_BYTES);
#pragma unroll
        for (int c = 0; c < Cfg::CH; ++c)
          tma_load_2d(sV + st * Cfg::TILE_BYTES + c * (F2_TILE * 128), &tmV, &v_full[st], hk * HD + c * 64,
                      row_base + j * F2_TILE);
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_qk = umma_idesc_bf16(F2_TILE, F2_TILE, 0, 0);
      constexpr uint32_t idesc_pv = umma_idesc_bf16(F2_TILE, HD, 0, 1);
      bool ok = mbar_wait(q_full, 0);
      if (!ok && p.status) atomicCAS(p.status, 0, GF_ERR_WAIT_FULL);
      const uint32_t ka = smem_u32(sK);
      for (int j = 0; j < n_j && ok; ++j) {
        if (!mbar_wait(k_full, j & 1)) {
          if (p.status) atomicCAS(p.status, 0, GF_ERR_WAIT_FULL);
          ok = false;
          break;
        }
#pragma unroll
        for (int t = 0; t < 2; ++t) {
          if (j >= n_kv[t]) continue;
          if (!mbar_wait(&s_empty[t], (j & 1) ^ 1)) {
            if (p.status) atomicCAS(p.status, 0, GF_ERR_WAIT_SOFTMAX);
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t qa = smem_u32(sQ + t * Cfg::TILE_BYTES);
#pragma unroll
          for (int kk = 0; kk < HD / 16; ++kk) {
            const uint32_t off = (kk >> 2) * (F2_TILE * 128) + (kk & 3) * 32;
            umma_bf16_ss(tmem_base + Cfg::TM_S + t * 128, umma_desc_sw128(qa + off, 16, 1024),
                         umma_desc_sw128(ka + off, 16, 1024), idesc_qk, kk > 0 ? 1u : 0u);
          }
          umma_commit(&s_full[t]);
        }
        if (!ok) break;
        umma_commit(k_empty);
        const int st = j & 1;
        if (!mbar_wait(&v_full[st], (j >> 1) & 1)) {
          if (p.status) atomicCAS(p.status, 0, GF_ERR_WAIT_FULL);
          ok = false;
          break;
        }
        const uint32_t va = smem_u32(sV + st * Cfg::TILE_BYTES);
#pragma unroll
        for (int t = 0; t < 2; ++t) {
          if (j >= n_kv[t]) continue;
          if (!mbar_wait(&p_full[t], j & 1)) {
            if (p.status) atomicCAS(p.status, 0, GF_ERR_WAIT_SOFTMAX);
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t pa = smem_u32(sP + t * Cfg::P_BYTES);
#pragma unroll
          for (int kk = 0; kk < F2_TILE / 16; ++kk) {
            const uint32_t aoff = (kk >> 2) * (F2_TILE * 128) + (kk & 3) * 32;
            umma_bf16_ss(tmem_base + Cfg::TM_O + t * 128, umma_desc_sw128(pa + aoff, 16, 1024),
                         umma_desc_sw128(va + kk * 2048, F2_TILE * 128, 1024), idesc_pv,
                         (j > 0 || kk > 0) ? 1u : 0u);
          }
          umma_commit(&pv_done[t]);
        }
        if (!ok) break;
        umma_commit(&v_empty[st]);
      }
    }
  } else {
    // ---------------------------------------------------------------- softmax warps: tile t = (warp - 2) / 4
    const int t = (warp - 2) >> 2;
    const int lane_grp = warp & 3;
    const int r = lane_grp * 32 + lane;
    const int q_idx = qb * 2 * F2_TILE + t * F2_TILE + r;
    const uint32_t tlane = (uint32_t)(lane_grp * 32) << 16;
    const uint32_t ts = tmem_base + Cfg::TM_S + t * 128 + tlane;
    const uint32_t to = tmem_base + Cfg::TM_O + t * 128 + tlane;
    const float sl2 = p.scale * 1.4426950408889634f;
    uint8_t* sPt = sP + t * Cfg::P_BYTES;
    float m_ref = -INFINITY, l = 0.f;
    bool ok = true;
    const int my_n = n_kv[t];
    for (int j = 0; j < my_n && ok; ++j) {
      if (!mbar_wait_warp(&s_full[t], j & 1)) {
        if (p.status) atomicCAS(p.status, 0, GF_ERR_WAIT_TMEM_FULL);
        ok = false;
        break;
      }
      tc_fence_after();
      const int kv0 = j * F2_TILE;
      const bool need_mask = (p.causal && (kv0 + F2_TILE - 1 > qb * 2 * F2_TILE + t * F2_TILE)) ||
                             (kv0 + F2_TILE > p.S);
      // ---- pass 1: row maximum of the raw scores
      float mx = -INFINITY;
      if (!need_mask) {
#pragma unroll
        for (int c = 0; c < F2_TILE / 32; ++c) {
          uint32_t rr[32];
          tmem_ld32(ts + c * 32, rr);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; i += 2)
            mx = fmaxf(mx, fmaxf(__uint_as_float(rr[i]), __uint_as_float(rr[i + 1])));
        }
      } else {
#pragma unroll
        for (int c = 0; c < F2_TILE / 32; ++c) {
          uint32_t rr[32];
          tmem_ld32(ts + c * 32, rr);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int kv = kv0 + c * 32 + i;
            const bool dead = kv >= p.S || (p.causal && kv > q_idx);
            mx = fmaxf(mx, dead ? -INFINITY : __uint_as_float(rr[i]));
          }
        }
      }
      // ---- reference maximum: move it (and rescale O, l) only when the row maximum grew a lot
      if (j == 0) {
        m_ref = mx;
      } else {
        const bool grow = (mx - m_ref) * sl2 > F2_RESCALE_THRESHOLD;
        // P(j) overwrites the shared-memory tile that P V (j-1) reads, and a rescale touches O:
        // both need P V (j-1) to have finished.
        if (!mbar_wait_warp(&pv_done[t], (j - 1) & 1)) {
          if (p.status) atomicCAS(p.status, 0, GF_ERR_WAIT_TMEM_FULL);
          ok = false;
          break;
        }
        if (__any_sync(0xffffffffu, grow)) {
          tc_fence_after();
          const float alpha = grow ? ex2_approx((m_ref - mx) * sl2) : 1.f;
#pragma unroll
          for (int c = 0; c < HD / 32; ++c) {
            uint32_t rr[32];
            tmem_ld32(to + c * 32, rr);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) rr[i] = __float_as_uint(__uint_as_float(rr[i]) * alpha);
            tmem_st32(to + c * 32, rr);
          }
          tmem_st_wait();
          l *= alpha;
          if (grow) m_ref = mx;
        }
      }
      const float mref_use = (m_ref == -INFINITY) ? 0.f : m_ref;  // row with no visible key yet
      const float mneg = -mref_use * sl2;
      // ---- pass 2: P = 2^(s*scale*log2e - m_ref*scale*log2e), bf16, into swizzled shared memory
      float rs = 0.f;
#pragma unroll
      for (int c = 0; c < F2_TILE / 32; ++c) {
        uint32_t rr[32];
        tmem_ld32(ts + c * 32, rr);
        tmem_ld_wait();
        uint32_t pk[16];
        if (!need_mask) {
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            const float p0 = ex2_approx(fmaf(__uint_as_float(rr[i]), sl2, mneg));
            const float p1 = ex2_approx(fmaf(__uint_as_float(rr[i + 1]), sl2, mneg));
            rs += p0 + p1;
            pk[i >> 1] = pack_bf16x2(p0, p1);
          }
        } else {
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            const int kv = kv0 + c * 32 + i;
            const bool d0 = kv >= p.S || (p.causal && kv > q_idx);
            const bool d1 = kv + 1 >= p.S || (p.causal && kv + 1 > q_idx);
            const float p0 = d0 ? 0.f : ex2_approx(fmaf(__uint_as_float(rr[i]), sl2, mneg));
            const float p1 = d1 ? 0.f : ex2_approx(fmaf(__uint_as_float(rr[i + 1]), sl2, mneg));
            rs += p0 + p1;
            pk[i >> 1] = pack_bf16x2(p0, p1);
          }
        }
        uint8_t* chunk = sPt + (c >> 1) * (F2_TILE * 128);
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          const uint32_t c16 = (uint32_t)((c & 1) * 4 + q4);
          *reinterpret_cast<uint4*>(chunk + sw128_offset((uint32_t)r, c16)) =
              make_uint4(pk[q4 * 4], pk[q4 * 4 + 1], pk[q4 * 4 + 2], pk[q4 * 4 + 3]);
        }
      }
      l += rs;
      tc_fence_before();
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&s_empty[t]);
        mbar_arrive(&p_full[t]);
      }
    }
    // ---- epilogue: O / l
    if (ok && my_n > 0) {
      if (!mbar_wait_warp(&pv_done[t], (my_n - 1) & 1)) {
        if (p.status) atomicCAS(p.status, 0, GF_ERR_WAIT_TMEM_FULL);
      } else {
        tc_fence_after();
        const float inv = l > 0.f ? 1.f / l : 0.f;
        __nv_bfloat16* orow = p.O + (long long)(row_base + q_idx) * p.ldo + h * HD;
#pragma unroll
        for (int c = 0; c < HD / 32; ++c) {
          uint32_t rr[32];
          tmem_ld32(to + c * 32, rr);
          tmem_ld_wait();
          if (q_idx < p.S) {
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4) {
              uint4 u;
              uint32_t* pu = reinterpret_cast<uint32_t*>(&u);
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const int i = q4 * 8 + e * 2;
                pu[e] = pack_bf16x2(__uint_as_float(rr[i]) * inv, __uint_as_float(rr[i + 1]) * inv);
              }
              *reinterpret_cast<uint4*>(orow + c * 32 + q4 * 8) = u;
            }
          }
        }
        if (q_idx < p.S && p.lse)
          p.lse[((long long)b * p.Hq + h) * p.S + q_idx] = m_ref * p.scale + logf(l);
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

template <int HD>
static int launch_fa2(const void* q, const void* k, const void* v, long long ldq, long long ldk, long long ldv,
                      Fa2Params& p, cudaStream_t stream) {
  using Cfg = Fa2Cfg<HD>;
  static gf::DeviceOnce configured;
  auto kern = fa_fwd2_kernel<HD>;
  if (configured.todo()) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES) != cudaSuccess)
      return GFH_CUDA;
    configured.mark();
  }
  const uint64_t T = (uint64_t)p.B * p.S;
  CUtensorMap tq, tk, tv;
  int rc = make_tmap_2d(&tq, q, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, T, (uint64_t)p.Hq * HD, ldq * 2, F2_TILE, 64);
  if (rc) return rc;
  rc = make_tmap_2d(&tk, k, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, T, (uint64_t)p.Hkv * HD, ldk * 2, F2_TILE, 64);
  if (rc) return rc;
  rc = make_tmap_2d(&tv, v, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, T, (uint64_t)p.Hkv * HD, ldv * 2, F2_TILE, 64);
  if (rc) return rc;
  dim3 grid((p.S + 2 * F2_TILE - 1) / (2 * F2_TILE), p.Hq, p.B);
  kern<<<grid, F2_THREADS, Cfg::SMEM_BYTES, stream>>>(tq, tk, tv, p);
  return cudaGetLastError() == cudaSuccess ? GFH_OK : GFH_CUDA;
}

}  // namespace gf

// Same contract as gf_flash_attn_fwd (attn_fwd.cu).
GF_API int gf_flash_attn_fwd2(const void* q, const void* k, const void* v, void* o, float* lse, int B, int S, int Hq,
                              int Hkv, int head_dim, long long ldq, long long ldk, long long ldv, long long ldo,
                              float scale, int causal, int* status, void* stream) {
  using namespace gf;
  enter();
  if (B <= 0 || S <= 0 || Hq <= 0 || Hkv <= 0 || Hq % Hkv) return GFH_BAD_ARG;
  if ((ldq % 8) || (ldk % 8) || (ldv % 8) || (ldo % 8)) return GFH_BAD_ARG;
  Fa2Params p;
  p.B = B; p.S = S; p.Hq = Hq; p.Hkv = Hkv; p.causal = causal; p.scale = scale;
  p.O = (__nv_bfloat16*)o; p.ldo = ldo; p.lse = lse; p.status = status;
  if (head_dim == 128) return launch_fa2<128>(q, k, v, ldq, ldk, ldv, p, (cudaStream_t)stream);
  if (head_dim == 64) return launch_fa2<64>(q, k, v, ldq, ldk, ldv, p, (cudaStream_t)stream);
  return GFH_BAD_ARG;
}
