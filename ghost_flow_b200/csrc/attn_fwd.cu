// FlashAttention forward for sm_100a: S = Q K^T and P V both run on tcgen05 with TMEM
// accumulators; Q/K/V tiles arrive by TMA straight out of the packed projection output
// (strided [tokens, heads*head_dim] views, no transposes); four softmax warps own one query
// row each, so row max/sum need no shuffles. Causal masking skips whole KV tiles above the
// diagonal; grouped-query attention maps query head h to KV head h / (Hq / Hkv).
//
// Replaces the reference's "fused_attention_kernel" (ghostflow-cuda/src/optimized_kernels.cu:185-248,
// one thread per query row, S <= 256, no mask) and the CPU tiled online-softmax forward
// (ghostflow-nn/src/flash_attention.rs:122-250).
#include "gf_host.h"
#include "gf_ptx.cuh"

namespace gf {

constexpr int FA_BM = 128;   // query rows per CTA
constexpr int FA_BN = 128;   // kv rows per tile
constexpr int FA_THREADS = 192;

struct FaFwdParams {
  int B, S, Hq, Hkv;
  int causal;
  float scale;          // applied to Q K^T
  __nv_bfloat16* O;
  long long ldo;
  float* lse;           // [B, Hq, S], natural log
  int* status;
};

template <int HD>
struct FaFwdCfg {
  static constexpr int CH = HD / 64;                      // 64-column chunks per row
  static constexpr int Q_BYTES = FA_BM * HD * 2;
  static constexpr int KV_BYTES = FA_BN * HD * 2;
  static constexpr int P_BYTES = FA_BM * FA_BN * 2;
  static constexpr int OFF_Q = 0;
  static constexpr int OFF_K = Q_BYTES;
  static constexpr int OFF_V = OFF_K + 2 * KV_BYTES;
  static constexpr int OFF_P = OFF_V + 2 * KV_BYTES;
  static constexpr int OFF_BAR = OFF_P + P_BYTES;
  static constexpr int SMEM_BYTES = OFF_BAR + 256 + 1024;
  static constexpr int TMEM_COLS = 512;                   // S0,S1 (128 each) + PV0,PV1 (HD each, <= 128)
  static constexpr int TM_S = 0;
  static constexpr int TM_PV = 256;
};

template <int HD>
__global__ void __launch_bounds__(FA_THREADS, 1)
fa_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
              const __grid_constant__ CUtensorMap tmV, const FaFwdParams p) {
  using Cfg = FaFwdCfg<HD>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem + Cfg::OFF_Q;
  uint8_t* sK = smem + Cfg::OFF_K;
  uint8_t* sV = smem + Cfg::OFF_V;
  uint8_t* sP = smem + Cfg::OFF_P;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::OFF_BAR);
  uint64_t* q_full = bars + 0;
  uint64_t* k_full = bars + 1;    // [2]
  uint64_t* k_empty = bars + 3;   // [2]
  uint64_t* v_full = bars + 5;    // [2]
  uint64_t* v_empty = bars + 7;   // [2]
  uint64_t* s_full = bars + 9;    // [2]
  uint64_t* s_empty = bars + 11;  // [2]
  uint64_t* p_full = bars + 13;
  uint64_t* p_empty = bars + 14;
  uint64_t* pv_full = bars + 15;  // [2]
  uint64_t* pv_empty = bars + 17; // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 19);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_qt = (p.S + FA_BM - 1) / FA_BM;
  const int qt = n_qt - 1 - (int)blockIdx.x;  // heaviest (last) query tiles first
  const int h = blockIdx.y, b = blockIdx.z;
  const int hk = h / (p.Hq / p.Hkv);
  const int n_kv_all = (p.S + FA_BN - 1) / FA_BN;
  const int n_kv = p.causal ? min(qt + 1, n_kv_all) : n_kv_all;
  const int row_base = b * p.S;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&s_empty[i], 4);
      mbar_init(&pv_full[i], 1);
      mbar_init(&pv_empty[i], 4);
    }
    mbar_init(p_full, 4);
    mbar_init(p_empty, 1);
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
      mbar_expect_tx(q_full, Cfg::Q_BYTES);
#pragma unroll
      for (int c = 0; c < Cfg::CH; ++c)
        tma_load_2d(sQ + c * (FA_BM * 128), &tmQ, q_full, h * HD + c * 64, row_base + qt * FA_BM);
      for (int j = 0; j < n_kv; ++j) {
        const int st = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!mbar_wait(&k_empty[st], ph ^ 1)) {
          if (p.status) atomicCAS(p.status, 0, GF_ERR_WAIT_EMPTY);
          break;
        }
        mbar_expect_tx(&k_full[st], Cfg::KV_BYTES);
#pragma unroll
        for (int c = 0; c < Cfg::CH; ++c)
          tma_load_2d(sK + st * Cfg::KV_BYTES + c * (FA_BN * 128), &tmK, &k_full[st], hk * HD + c * 64,
                      row_base + j * FA_BN);
        if (!mbar_wait(&v_empty[st], ph ^ 1)) {
          if (p.status) atomicCAS(p.status, 0, GF_ERR_WAIT_EMPTY);
          break;
        }
        mbar_expect_tx(&v_full[st], Cfg::KV_BYTES);
#pragma unroll
        for (int c = 0; c < Cfg::CH; ++c)
          tma_load_2d(sV + st * Cfg::KV_BYTES + c * (FA_BN * 128), &tmV, &v_full[st], hk * HD + c * 64,
                      row_base + j * FA_BN);
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_qk = umma_idesc_bf16(FA_BM, FA_BN, 0, 0);
      constexpr uint32_t idesc_pv = umma_idesc_bf16(FA_BM, HD, 0, 1);
      bool ok = mbar_wait(q_full, 0);
      if (!ok && p.status) atomicCAS(p.status, 0, GF_ERR_WAIT_FULL);
      auto issue_qk = [&](int j) -> bool {
        const int st = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!mbar_wait(&k_full[st], ph) || !mbar_wait(&s_empty[st], ph ^ 1)) {
          if (p.status) atomicCAS(p.status, 0, GF_ERR_WAIT_FULL);
          return false;
        }
        tc_fence_after();
        const uint32_t qa = smem_u32(sQ), ka = smem_u32(sK + st * Cfg::KV_BYTES);
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint32_t off = (kk >> 2) * (FA_BM * 128) + (kk & 3) * 32;
          umma_bf16_ss(tmem_base + Cfg::TM_S + st * FA_BN, umma_desc_sw128(qa + off, 16, 1024),
                       umma_desc_sw128(ka + off, 16, 1024), idesc_qk, kk > 0 ? 1u : 0u);
        }
        umma_commit(&k_empty[st]);
        umma_commit(&s_full[st]);
        return true;
      };
      if (ok) ok = issue_qk(0);
      for (int j = 0; j < n_kv && ok; ++j) {
        if (j + 1 < n_kv) {
          ok = issue_qk(j + 1);
          if (!ok) break;
        }
        const int st = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!mbar_wait(&v_full[st], ph) || !mbar_wait(p_full, j & 1) || !mbar_wait(&pv_empty[st], ph ^ 1)) {
          if (p.status) atomicCAS(p.status, 0, GF_ERR_WAIT_SOFTMAX);
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t pa = smem_u32(sP), va = smem_u32(sV + st * Cfg::KV_BYTES);
#pragma unroll
        for (int kk = 0; kk < FA_BN / 16; ++kk) {
          const uint32_t aoff = (kk >> 2) * (FA_BM * 128) + (kk & 3) * 32;
          umma_bf16_ss(tmem_base + Cfg::TM_PV + st * 128, umma_desc_sw128(pa + aoff, 16, 1024),
                       umma_desc_sw128(va + kk * 2048, FA_BN * 128, 1024), idesc_pv, kk > 0 ? 1u : 0u);
        }
        umma_commit(&v_empty[st]);
        umma_commit(p_empty);
        umma_commit(&pv_full[st]);
      }
    }
  } else {
    // ---------------------------------------------------------------- softmax + output (warps 2..5)
    const int lane_grp = warp & 3;
    const int r = lane_grp * 32 + lane;          // query row inside the tile
    const int q_idx = qt * FA_BM + r;            // position inside the sequence
    const uint32_t tlane = (uint32_t)(lane_grp * 32) << 16;
    const float sl2 = p.scale * 1.4426950408889634f;
    float o[HD];
#pragma unroll
    for (int i = 0; i < HD; ++i) o[i] = 0.f;
    float m = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; j < n_kv && ok; ++j) {
      const int st = j & 1;
      const uint32_t ph = (j >> 1) & 1;
      if (!mbar_wait_warp(&s_full[st], ph)) {
        if (p.status) atomicCAS(p.status, 0, GF_ERR_WAIT_TMEM_FULL);
        ok = false;
        break;
      }
      tc_fence_after();
      const uint32_t ts = tmem_base + Cfg::TM_S + st * FA_BN + tlane;
      const bool need_mask = (p.causal && j == qt) || ((j + 1) * FA_BN > p.S);
      const int kv0 = j * FA_BN;
      // pass 1: row max
      float mx = m;
#pragma unroll
      for (int c = 0; c < FA_BN / 32; ++c) {
        uint32_t rr[32];
        tmem_ld32(ts + c * 32, rr);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          float s = __uint_as_float(rr[i]);
          if (need_mask) {
            const int kv = kv0 + c * 32 + i;
            if (kv >= p.S || (p.causal && kv > q_idx)) s = -INFINITY;
          }
          mx = fmaxf(mx, s);
        }
      }
      const float m_new = mx;
      const float m_use = (m_new == -INFINITY) ? 0.f : m_new;  // fully masked row (only beyond S)
      const float alpha = exp2f((m - m_use) * sl2);
      // P(j) goes to shared memory once the previous P V product has been consumed
      if (!mbar_wait_warp(p_empty, (j & 1) ^ 1)) {
        if (p.status) atomicCAS(p.status, 0, GF_ERR_WAIT_SOFTMAX);
        ok = false;
        break;
      }
      float rs = 0.f;
#pragma unroll
      for (int c = 0; c < FA_BN / 32; ++c) {
        uint32_t rr[32];
        tmem_ld32(ts + c * 32, rr);
        tmem_ld_wait();
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float s0 = __uint_as_float(rr[i]), s1 = __uint_as_float(rr[i + 1]);
          if (need_mask) {
            const int kv = kv0 + c * 32 + i;
            if (kv >= p.S || (p.causal && kv > q_idx)) s0 = -INFINITY;
            if (kv + 1 >= p.S || (p.causal && kv + 1 > q_idx)) s1 = -INFINITY;
          }
          const float p0 = exp2f((s0 - m_use) * sl2), p1 = exp2f((s1 - m_use) * sl2);
          pk[i >> 1] = pack_bf16x2(p0, p1);
          // accumulate the row sum from the bf16-rounded values that the tensor core will see
          float2 pr = unpack_bf16x2(pk[i >> 1]);
          rs += pr.x + pr.y;
        }
        uint8_t* chunk = sP + (c >> 1) * (FA_BM * 128);
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          const uint32_t c16 = (uint32_t)((c & 1) * 4 + q4);
          *reinterpret_cast<uint4*>(chunk + sw128_offset((uint32_t)r, c16)) =
              make_uint4(pk[q4 * 4], pk[q4 * 4 + 1], pk[q4 * 4 + 2], pk[q4 * 4 + 3]);
        }
      }
      tc_fence_before();
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&s_empty[st]);
        mbar_arrive(p_full);
      }
      // fold the previous tile's P V into the running output, then rescale to the new max
      if (j > 0) {
        const int pst = (j - 1) & 1;
        if (!mbar_wait_warp(&pv_full[pst], ((j - 1) >> 1) & 1)) {
          if (p.status) atomicCAS(p.status, 0, GF_ERR_WAIT_TMEM_FULL);
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t tp = tmem_base + Cfg::TM_PV + pst * 128 + tlane;
#pragma unroll
        for (int c = 0; c < HD / 32; ++c) {
          uint32_t rr[32];
          tmem_ld32(tp + c * 32, rr);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[c * 32 + i] = (o[c * 32 + i] + __uint_as_float(rr[i])) * alpha;
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&pv_empty[pst]);
      }
      l = l * alpha + rs;
      m = m_new;
    }
    if (ok && n_kv > 0) {
      const int pst = (n_kv - 1) & 1;
      if (!mbar_wait_warp(&pv_full[pst], ((n_kv - 1) >> 1) & 1)) {
        if (p.status) atomicCAS(p.status, 0, GF_ERR_WAIT_TMEM_FULL);
        ok = false;
      } else {
        tc_fence_after();
        const uint32_t tp = tmem_base + Cfg::TM_PV + pst * 128 + tlane;
        const float inv = l > 0.f ? 1.f / l : 0.f;
        __nv_bfloat16* orow = p.O + (long long)(row_base + q_idx) * p.ldo + h * HD;
#pragma unroll
        for (int c = 0; c < HD / 32; ++c) {
          uint32_t rr[32];
          tmem_ld32(tp + c * 32, rr);
          tmem_ld_wait();
          if (q_idx < p.S) {
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4) {
              uint4 u;
              uint32_t* pu = reinterpret_cast<uint32_t*>(&u);
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const int i = q4 * 8 + e * 2;
                pu[e] = pack_bf16x2((o[c * 32 + i] + __uint_as_float(rr[i])) * inv,
                                    (o[c * 32 + i + 1] + __uint_as_float(rr[i + 1])) * inv);
              }
              *reinterpret_cast<uint4*>(orow + c * 32 + q4 * 8) = u;
            }
          }
        }
        if (q_idx < p.S && p.lse)
          p.lse[((long long)b * p.Hq + h) * p.S + q_idx] = m * p.scale + logf(l);
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
static int launch_fa_fwd(const void* q, const void* k, const void* v, long long ldq, long long ldk, long long ldv,
                         FaFwdParams& p, cudaStream_t stream) {
  using Cfg = FaFwdCfg<HD>;
  static gf::DeviceOnce configured;
  auto kern = fa_fwd_kernel<HD>;
  if (configured.todo()) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES) != cudaSuccess)
      return GFH_CUDA;
    configured.mark();
  }
  const uint64_t T = (uint64_t)p.B * p.S;
  CUtensorMap tq, tk, tv;
  int rc = make_tmap_2d(&tq, q, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, T, (uint64_t)p.Hq * HD, ldq * 2, FA_BM, 64);
  if (rc) return rc;
  rc = make_tmap_2d(&tk, k, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, T, (uint64_t)p.Hkv * HD, ldk * 2, FA_BN, 64);
  if (rc) return rc;
  rc = make_tmap_2d(&tv, v, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, T, (uint64_t)p.Hkv * HD, ldv * 2, FA_BN, 64);
  if (rc) return rc;
  dim3 grid((p.S + FA_BM - 1) / FA_BM, p.Hq, p.B);
  kern<<<grid, FA_THREADS, Cfg::SMEM_BYTES, stream>>>(tq, tk, tv, p);
  return cudaGetLastError() == cudaSuccess ? GFH_OK : GFH_CUDA;
}

}  // namespace gf

// q: [B*S, Hq*HD] rows with pitch ldq (elements); k, v: [B*S, Hkv*HD]; o: [B*S, Hq*HD] pitch ldo;
// lse: fp32 [B, Hq, S] (may be null). head_dim 64 or 128.
GF_API int gf_flash_attn_fwd(const void* q, const void* k, const void* v, void* o, float* lse, int B, int S, int Hq,
                             int Hkv, int head_dim, long long ldq, long long ldk, long long ldv, long long ldo,
                             float scale, int causal, int* status, void* stream) {
  gf::enter();
  using namespace gf;
  if (B <= 0 || S <= 0 || Hq <= 0 || Hkv <= 0 || Hq % Hkv) return GFH_BAD_ARG;
  if ((ldq % 8) || (ldk % 8) || (ldv % 8) || (ldo % 8)) return GFH_BAD_ARG;
  FaFwdParams p;
  p.B = B; p.S = S; p.Hq = Hq; p.Hkv = Hkv; p.causal = causal; p.scale = scale;
  p.O = (__nv_bfloat16*)o; p.ldo = ldo; p.lse = lse; p.status = status;
  if (head_dim == 128) return launch_fa_fwd<128>(q, k, v, ldq, ldk, ldv, p, (cudaStream_t)stream);
  if (head_dim == 64) return launch_fa_fwd<64>(q, k, v, ldq, ldk, ldv, p, (cudaStream_t)stream);
  return GFH_BAD_ARG;
}
