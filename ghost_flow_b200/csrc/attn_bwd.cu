// FlashAttention backward for sm_100a, all five products on tcgen05 with TMEM accumulators.
//
// One CTA owns a 128-row KV tile of one KV head and walks the 64-row query tiles that can
// see it (all query heads of the GQA group), working on transposed tiles so that every MMA
// has M = 128 and each compute thread owns one KV row:
//     S^T  = K Q^T            dP^T = V dO^T
//     P^T  = exp(S^T*scale - lse)        dS^T = P^T * (dP^T - delta) * scale
//     dV  += P^T dO           dK  += dS^T Q          dQ^T = K^T dS^T   (fp32 atomics into dq_acc)
// dV and dK stay in TMEM for the whole CTA lifetime and are written once at the end.
// K, V, Q and dO tiles are TMA loads from the strided projection outputs; the same shared-memory
// tile is used K-major by one product and MN-major by another, so nothing is transposed in memory.
//
// The reference only names a backward kernel (ghostflow-cuda/src/kernels/mod.rs:82) and has no
// backward for its CPU flash attention (ghostflow-nn/src/flash_attention.rs).
#include "gf_host.h"
#include "gf_ptx.cuh"

namespace gf {

constexpr int FB_KV = 128;  // kv rows per CTA
constexpr int FB_Q = 64;    // query rows per step
constexpr int FB_THREADS = 320;  // TMA warp, MMA warp, 2 x 4 compute warps (each group owns 32 of the 64 query columns)

struct FaBwdParams {
  int B, S, Hq, Hkv;
  int causal;
  float scale;
  const float* lse;    // [B, Hq, S]
  const float* delta;  // [B, Hq, S]
  float* dq_acc;       // fp32 [B*S, Hq*HD] (zeroed by the launcher)
  __nv_bfloat16* dK;
  long long lddk;
  __nv_bfloat16* dV;
  long long lddv;
  int* status;
};

template <int HD>
struct FaBwdCfg {
  static constexpr int CH = HD / 64;
  static constexpr int KV_BYTES = FB_KV * HD * 2;     // K or V tile
  static constexpr int Q_BYTES = FB_Q * HD * 2;       // Q or dO tile
  static constexpr int PT_BYTES = FB_KV * FB_Q * 2;   // P^T or dS^T tile (one 128-byte row per kv row)
  static constexpr int OFF_K = 0;
  static constexpr int OFF_V = OFF_K + KV_BYTES;
  static constexpr int OFF_Q = OFF_V + KV_BYTES;            // 2 stages
  static constexpr int OFF_DO = OFF_Q + 2 * Q_BYTES;        // 2 stages
  static constexpr int OFF_P = OFF_DO + 2 * Q_BYTES;
  static constexpr int OFF_DS = OFF_P + PT_BYTES;
  static constexpr int OFF_STAT = OFF_DS + PT_BYTES;        // 2 stages x (lse[64], delta[64]) fp32
  static constexpr int OFF_BAR = OFF_STAT + 2 * 2 * FB_Q * 4;
  static constexpr int SMEM_BYTES = OFF_BAR + 256 + 1024;
  static constexpr int STAGE_TX = 2 * Q_BYTES + 2 * FB_Q * 4;
  // TMEM columns
  static constexpr int TM_S = 0;      // 64
  static constexpr int TM_DP = 64;    // 64
  static constexpr int TM_DV = 128;   // HD
  static constexpr int TM_DK = 256;   // HD
  static constexpr int TM_DQ = 384;   // 2 x 64
  static constexpr int TMEM_COLS = 512;
};

__device__ __forceinline__ void bulk_load_1d(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(smem_dst)),
               "l"(reinterpret_cast<uint64_t>(gsrc)), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

template <int HD>
__global__ void __launch_bounds__(FB_THREADS, 1)
fa_bwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
              const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO,
              const FaBwdParams p) {
  using Cfg = FaBwdCfg<HD>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = smem + Cfg::OFF_K;
  uint8_t* sV = smem + Cfg::OFF_V;
  uint8_t* sQ = smem + Cfg::OFF_Q;
  uint8_t* sDO = smem + Cfg::OFF_DO;
  uint8_t* sP = smem + Cfg::OFF_P;
  uint8_t* sDS = smem + Cfg::OFF_DS;
  float* sStat = reinterpret_cast<float*>(smem + Cfg::OFF_STAT);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::OFF_BAR);
  uint64_t* kv_full = bars + 0;
  uint64_t* q_full = bars + 1;     // [2]
  uint64_t* q_empty = bars + 3;    // [2]
  uint64_t* s_full = bars + 5;
  uint64_t* s_empty = bars + 6;
  uint64_t* pds_full = bars + 7;
  uint64_t* pds_empty = bars + 8;
  uint64_t* dq_full = bars + 9;    // [2]
  uint64_t* dq_empty = bars + 11;  // [2]
  uint64_t* acc_full = bars + 13;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 14);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int j = blockIdx.x;  // kv tile
  const int hk = blockIdx.y, b = blockIdx.z;
  const int G = p.Hq / p.Hkv;
  const int n_q = p.S / FB_Q;
  const int i_start = p.causal ? (j * FB_KV) / FB_Q : 0;
  const int per_head = n_q - i_start;
  const int n_iter = G * per_head;
  const int row_base = b * p.S;

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&q_full[i], 1);
      mbar_init(&q_empty[i], 1);
    }
    mbar_init(s_full, 1);
    mbar_init(s_empty, 8);
    mbar_init(pds_full, 8);
    mbar_init(pds_empty, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&dq_full[i], 1);
      mbar_init(&dq_empty[i], 8);
    }
    mbar_init(acc_full, 1);
    mbar_fence_init();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
    tma_prefetch_desc(&tmDO);
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
      mbar_expect_tx(kv_full, 2 * Cfg::KV_BYTES);
#pragma unroll
      for (int c = 0; c < Cfg::CH; ++c) {
        tma_load_2d(sK + c * (FB_KV * 128), &tmK, kv_full, hk * HD + c * 64, row_base + j * FB_KV);
        tma_load_2d(sV + c * (FB_KV * 128), &tmV, kv_full, hk * HD + c * 64, row_base + j * FB_KV);
      }
      for (int it = 0; it < n_iter; ++it) {
        const int st = it & 1;
        const uint32_t ph = (it >> 1) & 1;
        const int h = hk * G + it / per_head;
        const int i = i_start + it % per_head;
        if (!mbar_wait(&q_empty[st], ph ^ 1)) {
          if (p.status) atomicCAS(p.status, 0, GF_ERR_WAIT_EMPTY);
          break;
        }
        mbar_expect_tx(&q_full[st], Cfg::STAGE_TX);
#pragma unroll
        for (int c = 0; c < Cfg::CH; ++c) {
          tma_load_2d(sQ + st * Cfg::Q_BYTES + c * (FB_Q * 128), &tmQ, &q_full[st], h * HD + c * 64,
                      row_base + i * FB_Q);
          tma_load_2d(sDO + st * Cfg::Q_BYTES + c * (FB_Q * 128), &tmDO, &q_full[st], h * HD + c * 64,
                      row_base + i * FB_Q);
        }
        const long long soff = ((long long)b * p.Hq + h) * p.S + (long long)i * FB_Q;
        bulk_load_1d(sStat + st * 2 * FB_Q, p.lse + soff, FB_Q * 4, &q_full[st]);
        bulk_load_1d(sStat + st * 2 * FB_Q + FB_Q, p.delta + soff, FB_Q * 4, &q_full[st]);
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_s = umma_idesc_bf16(128, FB_Q, 0, 0);    // S^T, dP^T
      constexpr uint32_t idesc_acc = umma_idesc_bf16(128, HD, 0, 1);    // dV, dK
      constexpr uint32_t idesc_dq = umma_idesc_bf16(128, FB_Q, 1, 1);   // dQ^T
      constexpr uint32_t K_LBO = FB_KV * 128;  // HD = 64: output rows 64..127 read the V tile, finite and never used
      const uint32_t ka = smem_u32(sK), va = smem_u32(sV), pa = smem_u32(sP), dsa = smem_u32(sDS);
      bool ok = mbar_wait(kv_full, 0);
      if (!ok && p.status) atomicCAS(p.status, 0, GF_ERR_WAIT_FULL);
      auto issue_s = [&](int it) -> bool {
        const int st = it & 1;
        if (!mbar_wait(&q_full[st], (it >> 1) & 1) || !mbar_wait(s_empty, (it & 1) ^ 1)) {
          if (p.status) atomicCAS(p.status, 0, GF_ERR_WAIT_FULL);
          return false;
        }
        tc_fence_after();
        const uint32_t qa = smem_u32(sQ + st * Cfg::Q_BYTES), doa = smem_u32(sDO + st * Cfg::Q_BYTES);
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint32_t aoff = (kk >> 2) * (FB_KV * 128) + (kk & 3) * 32;
          const uint32_t boff = (kk >> 2) * (FB_Q * 128) + (kk & 3) * 32;
          umma_bf16_ss(tmem_base + Cfg::TM_S, umma_desc_sw128(ka + aoff, 16, 1024),
                       umma_desc_sw128(qa + boff, 16, 1024), idesc_s, kk > 0 ? 1u : 0u);
        }
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint32_t aoff = (kk >> 2) * (FB_KV * 128) + (kk & 3) * 32;
          const uint32_t boff = (kk >> 2) * (FB_Q * 128) + (kk & 3) * 32;
          umma_bf16_ss(tmem_base + Cfg::TM_DP, umma_desc_sw128(va + aoff, 16, 1024),
                       umma_desc_sw128(doa + boff, 16, 1024), idesc_s, kk > 0 ? 1u : 0u);
        }
        umma_commit(s_full);
        return true;
      };
      if (ok) ok = issue_s(0);
      for (int it = 0; it < n_iter && ok; ++it) {
        if (it + 1 < n_iter) {
          ok = issue_s(it + 1);
          if (!ok) break;
        }
        const int st = it & 1;
        if (!mbar_wait(pds_full, it & 1) || !mbar_wait(&dq_empty[st], ((it >> 1) & 1) ^ 1)) {
          if (p.status) atomicCAS(p.status, 0, GF_ERR_WAIT_SOFTMAX);
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t qa = smem_u32(sQ + st * Cfg::Q_BYTES), doa = smem_u32(sDO + st * Cfg::Q_BYTES);
        // dV += P^T dO ; dK += dS^T Q   (K = 64 query rows -> 4 steps)
#pragma unroll
        for (int kk = 0; kk < FB_Q / 16; ++kk)
          umma_bf16_ss(tmem_base + Cfg::TM_DV, umma_desc_sw128(pa + kk * 32, 16, 1024),
                       umma_desc_sw128(doa + kk * 2048, FB_Q * 128, 1024), idesc_acc, (it > 0 || kk > 0) ? 1u : 0u);
#pragma unroll
        for (int kk = 0; kk < FB_Q / 16; ++kk)
          umma_bf16_ss(tmem_base + Cfg::TM_DK, umma_desc_sw128(dsa + kk * 32, 16, 1024),
                       umma_desc_sw128(qa + kk * 2048, FB_Q * 128, 1024), idesc_acc, (it > 0 || kk > 0) ? 1u : 0u);
        // dQ^T = K^T dS^T   (K = 128 kv rows -> 8 steps)
#pragma unroll
        for (int kk = 0; kk < FB_KV / 16; ++kk)
          umma_bf16_ss(tmem_base + Cfg::TM_DQ + st * FB_Q, umma_desc_sw128(ka + kk * 2048, K_LBO, 1024),
                       umma_desc_sw128(dsa + kk * 2048, FB_KV * 128, 1024), idesc_dq, kk > 0 ? 1u : 0u);
        umma_commit(&q_empty[st]);
        umma_commit(pds_empty);
        umma_commit(&dq_full[st]);
      }
      if (ok) umma_commit(acc_full);
    }
  } else {
    // ---------------------------------------------------------------- compute warps (2..9)
    // Warps 2..5 own query columns 0..31 of S^T / dP^T / dQ^T, warps 6..9 own columns 32..63; within a
    // group, warp w owns TMEM lanes 32 * (w % 4) .. +31, one kv row (or one head-dim row of dQ^T) per thread.
    const int hf = (warp - 2) >> 2;
    const int lane_grp = warp & 3;
    const int r = lane_grp * 32 + lane;
    const int kv_idx = j * FB_KV + r;
    const uint32_t tlane = (uint32_t)(lane_grp * 32) << 16;
    const float sl2 = p.scale * 1.4426950408889634f;
    const float l2e = 1.4426950408889634f;
    const long long dq_ld = (long long)p.Hq * HD;
    bool ok = true;

    auto drain_dq = [&](int it) -> bool {
      if (!mbar_wait_warp(&dq_full[it & 1], (it >> 1) & 1)) {
        if (p.status) atomicCAS(p.status, 0, GF_ERR_WAIT_TMEM_FULL);
        return false;
      }
      tc_fence_after();
      const int h = hk * G + it / per_head;
      const int i = i_start + it % per_head;
      float* dst = p.dq_acc + (long long)(row_base + i * FB_Q + hf * 32) * dq_ld + h * HD + r;
      uint32_t rr[32];
      tmem_ld32(tmem_base + Cfg::TM_DQ + (it & 1) * FB_Q + hf * 32 + tlane, rr);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&dq_empty[it & 1]);
      if (r < HD) {
#pragma unroll
        for (int e = 0; e < 32; ++e) atomicAdd(dst + (long long)e * dq_ld, __uint_as_float(rr[e]));
      }
      return true;
    };

    for (int it = 0; it < n_iter && ok; ++it) {
      const int st = it & 1;
      const int i = i_start + it % per_head;
      if (!mbar_wait_warp(s_full, it & 1)) {
        if (p.status) atomicCAS(p.status, 0, GF_ERR_WAIT_TMEM_FULL);
        ok = false;
        break;
      }
      tc_fence_after();
      const float* lse_s = sStat + st * 2 * FB_Q + hf * 32;
      const float* del_s = lse_s + FB_Q;
      const int q0 = i * FB_Q + hf * 32;
      const bool diag = p.causal && (q0 < j * FB_KV + FB_KV);  // these columns touch the diagonal
      uint32_t pp[16], dd[16];
      {
        uint32_t sv[32], dpv[32];
        tmem_ld32(tmem_base + Cfg::TM_S + hf * 32 + tlane, sv);
        tmem_ld32(tmem_base + Cfg::TM_DP + hf * 32 + tlane, dpv);
        tmem_ld_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(s_empty);
        if (!diag) {
#pragma unroll
          for (int e = 0; e < 32; e += 2) {
            const float p0 = ex2_approx(fmaf(__uint_as_float(sv[e]), sl2, -lse_s[e] * l2e));
            const float p1 = ex2_approx(fmaf(__uint_as_float(sv[e + 1]), sl2, -lse_s[e + 1] * l2e));
            const float d0 = p0 * (__uint_as_float(dpv[e]) - del_s[e]) * p.scale;
            const float d1 = p1 * (__uint_as_float(dpv[e + 1]) - del_s[e + 1]) * p.scale;
            pp[e >> 1] = pack_bf16x2(p0, p1);
            dd[e >> 1] = pack_bf16x2(d0, d1);
          }
        } else {
#pragma unroll
          for (int e = 0; e < 32; e += 2) {
            float p0 = ex2_approx(fmaf(__uint_as_float(sv[e]), sl2, -lse_s[e] * l2e));
            float p1 = ex2_approx(fmaf(__uint_as_float(sv[e + 1]), sl2, -lse_s[e + 1] * l2e));
            if (q0 + e < kv_idx) p0 = 0.f;
            if (q0 + e + 1 < kv_idx) p1 = 0.f;
            const float d0 = p0 * (__uint_as_float(dpv[e]) - del_s[e]) * p.scale;
            const float d1 = p1 * (__uint_as_float(dpv[e + 1]) - del_s[e + 1]) * p.scale;
            pp[e >> 1] = pack_bf16x2(p0, p1);
            dd[e >> 1] = pack_bf16x2(d0, d1);
          }
        }
      }
      if (!mbar_wait_warp(pds_empty, (it & 1) ^ 1)) {
        if (p.status) atomicCAS(p.status, 0, GF_ERR_WAIT_SOFTMAX);
        ok = false;
        break;
      }
#pragma unroll
      for (int c4 = 0; c4 < 4; ++c4) {
        const uint32_t off = sw128_offset((uint32_t)r, (uint32_t)(hf * 4 + c4));
        *reinterpret_cast<uint4*>(sP + off) = make_uint4(pp[c4 * 4], pp[c4 * 4 + 1], pp[c4 * 4 + 2], pp[c4 * 4 + 3]);
        *reinterpret_cast<uint4*>(sDS + off) = make_uint4(dd[c4 * 4], dd[c4 * 4 + 1], dd[c4 * 4 + 2], dd[c4 * 4 + 3]);
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(pds_full);
      if (it > 0) ok = drain_dq(it - 1);
    }
    if (ok && n_iter > 0) ok = drain_dq(n_iter - 1);
    if (ok) {
      if (!mbar_wait_warp(acc_full, 0)) {
        if (p.status) atomicCAS(p.status, 0, GF_ERR_WAIT_TMEM_FULL);
      } else {
        tc_fence_after();
        __nv_bfloat16* dkr = p.dK + (long long)(row_base + kv_idx) * p.lddk + hk * HD;
        __nv_bfloat16* dvr = p.dV + (long long)(row_base + kv_idx) * p.lddv + hk * HD;
        // each group writes half of the head dimension
#pragma unroll
        for (int cc = 0; cc < HD / 64; ++cc) {
          const int c = hf * (HD / 64) + cc;
          uint32_t rk[32], rv[32];
          tmem_ld32(tmem_base + Cfg::TM_DK + c * 32 + tlane, rk);
          tmem_ld32(tmem_base + Cfg::TM_DV + c * 32 + tlane, rv);
          tmem_ld_wait();
          if (kv_idx < p.S) {
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4) {
              uint4 uk, uv;
              uint32_t* pk = reinterpret_cast<uint32_t*>(&uk);
              uint32_t* pv = reinterpret_cast<uint32_t*>(&uv);
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const int idx = q4 * 8 + e * 2;
                pk[e] = pack_bf16x2(__uint_as_float(rk[idx]), __uint_as_float(rk[idx + 1]));
                pv[e] = pack_bf16x2(__uint_as_float(rv[idx]), __uint_as_float(rv[idx + 1]));
              }
              *reinterpret_cast<uint4*>(dkr + c * 32 + q4 * 8) = uk;
              *reinterpret_cast<uint4*>(dvr + c * 32 + q4 * 8) = uv;
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

// delta[b,h,s] = sum_d O * dO ; one warp per (token, head).
__global__ void attn_bwd_prep_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ dout,
                                     float* __restrict__ delta, int B, int S, int Hq, int HD, long long ldo,
                                     long long lddo) {
  const long long gw = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const long long total = (long long)B * S * Hq;
  if (gw >= total) return;
  const int h = (int)(gw % Hq);
  const long long t = gw / Hq;
  const __nv_bfloat16* op = o + t * ldo + h * HD;
  const __nv_bfloat16* dp = dout + t * lddo + h * HD;
  float acc = 0.f;
  for (int d = lane * 2; d < HD; d += 64) {
    float2 a = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(op + d));
    float2 g = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(dp + d));
    acc += a.x * g.x + a.y * g.y;
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
  if (lane == 0) {
    const long long bb = t / S, s = t % S;
    delta[(bb * Hq + h) * S + s] = acc;
  }
}

__global__ void cast_f32_bf16_2d_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst, long long rows,
                                        int cols, long long lds, long long ldd, float scale) {
  const int vpr = cols >> 2;
  const long long total = rows * vpr;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long rrow = idx / vpr;
    const int v = (int)(idx % vpr);
    float4 f = *reinterpret_cast<const float4*>(src + rrow * lds + v * 4);
    uint2 o;
    o.x = pack_bf16x2(f.x * scale, f.y * scale);
    o.y = pack_bf16x2(f.z * scale, f.w * scale);
    *reinterpret_cast<uint2*>(dst + rrow * ldd + v * 4) = o;
  }
}

template <int HD>
static int launch_fa_bwd(const void* q, const void* k, const void* v, const void* dout, long long ldq, long long ldk,
                         long long ldv, long long lddo, FaBwdParams& p, cudaStream_t stream) {
  using Cfg = FaBwdCfg<HD>;
  static gf::DeviceOnce configured;
  auto kern = fa_bwd_kernel<HD>;
  if (configured.todo()) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES) != cudaSuccess)
      return GFH_CUDA;
    configured.mark();
  }
  const uint64_t T = (uint64_t)p.B * p.S;
  CUtensorMap tq, tk, tv, tdo;
  int rc = make_tmap_2d(&tq, q, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, T, (uint64_t)p.Hq * HD, ldq * 2, FB_Q, 64);
  if (rc) return rc;
  rc = make_tmap_2d(&tdo, dout, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, T, (uint64_t)p.Hq * HD, lddo * 2, FB_Q, 64);
  if (rc) return rc;
  rc = make_tmap_2d(&tk, k, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, T, (uint64_t)p.Hkv * HD, ldk * 2, FB_KV, 64);
  if (rc) return rc;
  rc = make_tmap_2d(&tv, v, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, T, (uint64_t)p.Hkv * HD, ldv * 2, FB_KV, 64);
  if (rc) return rc;
  dim3 grid(p.S / FB_KV, p.Hkv, p.B);
  kern<<<grid, FB_THREADS, Cfg::SMEM_BYTES, stream>>>(tq, tk, tv, tdo, p);
  return cudaGetLastError() == cudaSuccess ? GFH_OK : GFH_CUDA;
}

}  // namespace gf

using namespace gf;

GF_API int gf_attn_bwd_prep(const void* o, const void* dout, float* delta, float* dq_acc, int B, int S, int Hq,
                            int HD, long long ldo, long long lddo, void* stream) {
  gf::enter();
  const long long warps = (long long)B * S * Hq;
  const int threads = 256;
  const long long blocks = (warps * 32 + threads - 1) / threads;
  attn_bwd_prep_kernel<<<(unsigned)blocks, threads, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)o, (const __nv_bfloat16*)dout, delta, B, S, Hq, HD, ldo, lddo);
  if (dq_acc) cudaMemsetAsync(dq_acc, 0, (size_t)B * S * Hq * HD * sizeof(float), (cudaStream_t)stream);
  return cudaGetLastError() == cudaSuccess ? GFH_OK : GFH_CUDA;
}

// dq_acc: fp32 [B*S, Hq*HD] zero-initialised (gf_attn_bwd_prep does it); convert afterwards with
// gf_cast_f32_to_bf16_2d. S must be a multiple of 128.
GF_API int gf_flash_attn_bwd(const void* q, const void* k, const void* v, const void* dout, const float* lse,
                             const float* delta, float* dq_acc, void* dk, void* dv, int B, int S, int Hq, int Hkv,
                             int head_dim, long long ldq, long long ldk, long long ldv, long long lddo,
                             long long lddk, long long lddv, float scale, int causal, int* status, void* stream) {
  gf::enter();
  if (B <= 0 || S <= 0 || (S % FB_KV) || Hq % Hkv) return GFH_BAD_ARG;
  if ((ldq % 8) || (ldk % 8) || (ldv % 8) || (lddo % 8) || (lddk % 8) || (lddv % 8)) return GFH_BAD_ARG;
  FaBwdParams p;
  p.B = B; p.S = S; p.Hq = Hq; p.Hkv = Hkv; p.causal = causal; p.scale = scale;
  p.lse = lse; p.delta = delta; p.dq_acc = dq_acc;
  p.dK = (__nv_bfloat16*)dk; p.lddk = lddk; p.dV = (__nv_bfloat16*)dv; p.lddv = lddv; p.status = status;
  if (head_dim == 128) return launch_fa_bwd<128>(q, k, v, dout, ldq, ldk, ldv, lddo, p, (cudaStream_t)stream);
  if (head_dim == 64) return launch_fa_bwd<64>(q, k, v, dout, ldq, ldk, ldv, lddo, p, (cudaStream_t)stream);
  return GFH_BAD_ARG;
}

GF_API int gf_cast_f32_to_bf16_2d(const float* src, void* dst, long long rows, int cols, long long lds,
                                  long long ldd, float scale, void* stream) {
  gf::enter();
  if (cols % 4 || lds % 4 || ldd % 4) return GFH_BAD_ARG;
  long long total = rows * (cols / 4);
  long long g = (total + 255) / 256;
  const long long cap = (long long)sm_count() * 16;
  if (g > cap) g = cap;
  if (g < 1) g = 1;
  cast_f32_bf16_2d_kernel<<<(unsigned)g, 256, 0, (cudaStream_t)stream>>>(src, (__nv_bfloat16*)dst, rows, cols, lds,
                                                                        ldd, scale);
  return cudaGetLastError() == cudaSuccess ? GFH_OK : GFH_CUDA;
}
