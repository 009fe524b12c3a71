// FlashAttention backward, second generation. The products and tile shapes are those of attn_bwd.cu
// (one CTA owns a 128-row KV tile of one KV head and walks the 64-row query tiles that can see it; S^T, dP^T,
// dV, dK and dQ^T on tcgen05 with TMEM accumulators), reorganised so that no warp ever waits for work that
// is not its own:
//
//   * a fourth warpgroup does nothing but drain dQ^T from tensor memory, so the eight compute warps only turn
//     S^T / dP^T into P^T / dS^T. The drain warps transpose a half tile (32 query rows x HD) through shared memory
//     and hand it to the bulk-copy engine as ONE fp32 add-reduction (cp.reduce.async.bulk) into the accumulator,
//     which is laid out tile by tile ([B, Hq, S / 64, 64, HD]) so that a half tile is one contiguous block.
//     Per-thread red.global.add of the same data (8192 scalar atomics per step and SM) was the limit of the first kernel;
//   * tcgen05.mma fetches its shared-memory operands at about 64 bytes per clock, which is what bounds this kernel
//     (five products per step, about 200 KB of operand reads when everything sits in shared memory). P^T and dS^T
//     therefore go back into tensor memory as packed bf16, over the S^T / dP^T buffers they were computed from,
//     and dV += P^T dO, dK += dS^T Q take their A operand from there; only dQ^T = K^T dS^T, which needs dS^T as
//     its B operand, still reads a (double-buffered) shared-memory copy of dS^T;
//   * the softmax scale is taken out of the element loop (dS^T leaves unscaled; dK is scaled once in the
//     epilogue and dQ in the conversion kernel), and the row statistics arrive as -lse * log2(e), so one P / dS
//     pair costs an FMA, an exponential, a subtraction, a multiplication and two conversions;
//   * the statistics are read from shared memory sixteen bytes at a time;
//   * Q / dO tiles sit in three stages and the MMA warp polls its two kinds of work (the S^T / dP^T pair of the next
//     step, the dQ^T / dV / dK triple of the current one) without blocking on either, so a tile that is still
//     in flight never holds up products whose inputs are ready.
//
// The reference only names a backward kernel (ghostflow-cuda/src/kernels/mod.rs:82) and has no backward for its
// CPU flash attention (ghostflow-nn/src/flash_attention.rs).
#include "gf_host.h"
#include "gf_ptx.cuh"

namespace gf {

constexpr int B2_KV = 128;       // kv rows per CTA
constexpr int B2_Q = 64;         // query rows per step
constexpr int B2_QST = 3;        // Q / dO / statistics stages: a tile is requested two steps before its first use,
                                 // because a stage is only free once the dK product that read it has completed
constexpr int B2_THREADS = 512;  // warpgroup 0: TMA warp, MMA warp, two idle; 1 and 2: compute; 3: dQ drain

struct FaBwd2Params {
  int B, S, Hq, Hkv;
  int causal;
  float scale;
  const float* nlse2;  // [B, Hq, S]  -lse * log2(e)
  const float* delta;  // [B, Hq, S]
  float* dq_acc;       // fp32 [B, Hq, S / 64, 64, HD], zero before launch; receives dQ / scale
  __nv_bfloat16* dK;
  long long lddk;
  __nv_bfloat16* dV;
  long long lddv;
  int* status;
  int head_group;   // KV heads whose CTAs are dispatched together
};

template <int HD>
struct FaBwd2Cfg {
  static constexpr int CH = HD / 64;
  static constexpr int KV_BYTES = B2_KV * HD * 2;     // K or V tile
  static constexpr int Q_BYTES = B2_Q * HD * 2;       // Q or dO tile
  static constexpr int PT_BYTES = B2_KV * B2_Q * 2;   // P^T or dS^T tile (one 128-byte row per kv row)
  static constexpr int OFF_K = 0;
  static constexpr int OFF_V = OFF_K + KV_BYTES;
  static constexpr int OFF_Q = OFF_V + KV_BYTES;            // B2_QST stages
  static constexpr int OFF_DO = OFF_Q + B2_QST * Q_BYTES;   // B2_QST stages
  static constexpr int OFF_DS = OFF_DO + B2_QST * Q_BYTES;  // 2 buffers
  static constexpr int DQ_HALF_BYTES = (B2_Q / 2) * HD * 4; // staging of half a dQ tile: [32 query rows][HD] fp32
  static constexpr int OFF_DQS = OFF_DS + 2 * PT_BYTES;
  static constexpr int OFF_STAT = OFF_DQS + DQ_HALF_BYTES;  // B2_QST stages x (nlse2[64], delta[64]) fp32
  static constexpr int OFF_BAR = OFF_STAT + B2_QST * 2 * B2_Q * 4;
  static constexpr int SMEM_BYTES = OFF_BAR + 256 + 1024;
  static constexpr int STAGE_TX = 2 * Q_BYTES + 2 * B2_Q * 4;
  // TMEM columns. S^T and dP^T are double-buffered (buffer b = step & 1 at column b * 128). A compute warp that
  // owns query columns [32 hf, 32 hf + 32) of S^T writes its half of P^T (16 columns of bf16 pairs) over the
  // first 16 of them, likewise dS^T over dP^T; dQ^T of the step is then written over the whole dP^T buffer,
  // after dK has consumed dS^T (MMAs execute in issue order).
  static constexpr int TM_S = 0;      // + b * 128, 64 columns; P^T at [0, 16) and [32, 48) afterwards
  static constexpr int TM_DP = 64;    // + b * 128, 64 columns; dS^T likewise, then dQ^T
  static constexpr int TM_DV = 256;   // HD
  static constexpr int TM_DK = 384;   // HD
  static constexpr int TMEM_COLS = 512;
};

__device__ __forceinline__ void bulk_load_1d_b2(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(smem_dst)),
               "l"(reinterpret_cast<uint64_t>(gsrc)), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

template <int HD>
__global__ void __launch_bounds__(B2_THREADS, 1)
fa_bwd2_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
               const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO,
               const FaBwd2Params p) {
  using Cfg = FaBwd2Cfg<HD>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = smem + Cfg::OFF_K;
  uint8_t* sV = smem + Cfg::OFF_V;
  uint8_t* sQ = smem + Cfg::OFF_Q;
  uint8_t* sDO = smem + Cfg::OFF_DO;
  uint8_t* sDS = smem + Cfg::OFF_DS;
  float* sStat = reinterpret_cast<float*>(smem + Cfg::OFF_STAT);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::OFF_BAR);
  uint64_t* kv_full = bars + 0;
  uint64_t* acc_full = bars + 1;
  uint64_t* s_full = bars + 2;      // [2]
  uint64_t* pds_full = bars + 4;    // [2]
  uint64_t* pds_empty = bars + 6;   // [2]
  uint64_t* dq_full = bars + 8;     // [2]
  uint64_t* dq_empty = bars + 10;   // [2]
  uint64_t* s_empty = bars + 12;    // [2]
  uint64_t* q_full = bars + 14;     // [B2_QST]
  uint64_t* q_empty = q_full + B2_QST;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(q_empty + B2_QST);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // Linear block order: KV heads in groups of head_group; inside a group the heaviest KV tile of every head first
  // (under a causal mask tile 0 is seen by every query tile, the last one by two), so the CTAs in flight share the
  // Q / dO tiles of few heads in L2 and the short CTAs fill the tail.
  int j, hk;
  {
    const int H = gridDim.x, NT = gridDim.y;
    const int lin = blockIdx.x + H * blockIdx.y;
    const int gs = p.head_group;
    const int g = lin / (gs * NT);
    const int rem = lin - g * gs * NT;
    const int gs_g = min(gs, H - g * gs);
    j = rem / gs_g;
    hk = g * gs + rem % gs_g;
  }
  const int b = blockIdx.z;
  const int G = p.Hq / p.Hkv;
  const int n_q = p.S / B2_Q;
  const int i_start = p.causal ? (j * B2_KV) / B2_Q : 0;
  const int per_head = n_q - i_start;
  const int n_iter = G * per_head;
  const int row_base = b * p.S;

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int i = 0; i < B2_QST; ++i) {
      mbar_init(&q_full[i], 1);
      mbar_init(&q_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&pds_full[i], 8);
      mbar_init(&pds_empty[i], 1);
      mbar_init(&dq_full[i], 1);
      mbar_init(&dq_empty[i], 4);
      mbar_init(&s_full[i], 1);
      mbar_init(&s_empty[i], 8);
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
        tma_load_2d(sK + c * (B2_KV * 128), &tmK, kv_full, hk * HD + c * 64, row_base + j * B2_KV);
        tma_load_2d(sV + c * (B2_KV * 128), &tmV, kv_full, hk * HD + c * 64, row_base + j * B2_KV);
      }
      for (int it = 0; it < n_iter; ++it) {
        const int st = it % B2_QST;
        const uint32_t ph = (it / B2_QST) & 1;
        const int h = hk * G + it / per_head;
        const int i = i_start + it % per_head;
        if (!mbar_wait(&q_empty[st], ph ^ 1)) {
          if (p.status) atomicCAS(p.status, 0, GF_ERR_WAIT_EMPTY);
          break;
        }
        mbar_expect_tx(&q_full[st], Cfg::STAGE_TX);
#pragma unroll
        for (int c = 0; c < Cfg::CH; ++c) {
          tma_load_2d(sQ + st * Cfg::Q_BYTES + c * (B2_Q * 128), &tmQ, &q_full[st], h * HD + c * 64,
                      row_base + i * B2_Q);
          tma_load_2d(sDO + st * Cfg::Q_BYTES + c * (B2_Q * 128), &tmDO, &q_full[st], h * HD + c * 64,
                      row_base + i * B2_Q);
        }
        const long long soff = ((long long)b * p.Hq + h) * p.S + (long long)i * B2_Q;
        bulk_load_1d_b2(sStat + st * 2 * B2_Q, p.nlse2 + soff, B2_Q * 4, &q_full[st]);
        bulk_load_1d_b2(sStat + st * 2 * B2_Q + B2_Q, p.delta + soff, B2_Q * 4, &q_full[st]);
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    // The whole warp runs this code in uniform control flow; one elected lane issues (see gf_ptx.cuh).
    {
      const bool leader = elect_one();
      constexpr uint32_t idesc_s = umma_idesc_bf16(128, B2_Q, 0, 0);    // S^T, dP^T
      constexpr uint32_t idesc_acc = umma_idesc_bf16(128, HD, 0, 1);    // dV, dK
      constexpr uint32_t idesc_dq = umma_idesc_bf16(128, B2_Q, 1, 1);   // dQ^T
      constexpr uint32_t K_LBO = B2_KV * 128;  // HD = 64: output rows 64..127 read the V tile, finite and never used
      const uint32_t ka = smem_u32(sK), va = smem_u32(sV);
      bool ok = mbar_wait_warp(kv_full, 0);
      if (!ok && p.status && leader) atomicCAS(p.status, 0, GF_ERR_WAIT_FULL);
      // S^T(it) = K Q^T and dP^T(it) = V dO^T into buffer it & 1
      auto issue_s = [&](int it) {
        const int st = it % B2_QST;
        const uint32_t tb = tmem_base + (it & 1) * 128;
        tc_fence_after();
        const uint32_t qa = smem_u32(sQ + st * Cfg::Q_BYTES), doa = smem_u32(sDO + st * Cfg::Q_BYTES);
        // the two products accumulate into different TMEM buffers; alternating them keeps two independent
        // accumulation chains in the tensor pipe
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint32_t aoff = (kk >> 2) * (B2_KV * 128) + (kk & 3) * 32;
          const uint32_t boff = (kk >> 2) * (B2_Q * 128) + (kk & 3) * 32;
          umma_bf16_ss_u(leader, tb + Cfg::TM_S, umma_desc_sw128(ka + aoff, 16, 1024),
                       umma_desc_sw128(qa + boff, 16, 1024), idesc_s, kk > 0 ? 1u : 0u);
          umma_bf16_ss_u(leader, tb + Cfg::TM_DP, umma_desc_sw128(va + aoff, 16, 1024),
                       umma_desc_sw128(doa + boff, 16, 1024), idesc_s, kk > 0 ? 1u : 0u);
        }
        umma_commit_u(leader, &s_full[it & 1]);
      };
      // dQ^T(it), dV += , dK += from P^T(it) / dS^T(it)
      auto issue_grads = [&](int it) {
        const int st = it % B2_QST, pb = it & 1;
        tc_fence_after();
        const uint32_t qa = smem_u32(sQ + st * Cfg::Q_BYTES), doa = smem_u32(sDO + st * Cfg::Q_BYTES);
        const uint32_t dsa = smem_u32(sDS + pb * Cfg::PT_BYTES);
        const uint32_t tP = tmem_base + pb * 128 + Cfg::TM_S, tdS = tmem_base + pb * 128 + Cfg::TM_DP;
        // dV += P^T dO and dK += dS^T Q (K = 64 query rows -> 4 steps each), A operands from tensor memory: k step kk
        // covers query columns 16 kk .., i.e. columns 8 (kk & 1) of the half (kk >> 1) that starts at 32 (kk >> 1).
        // Two independent accumulators, issued alternately.
#pragma unroll
        for (int kk = 0; kk < B2_Q / 16; ++kk) {
          const uint32_t acol = (uint32_t)((kk >> 1) * 32 + (kk & 1) * 8);
          umma_bf16_ts_u(leader, tmem_base + Cfg::TM_DV, tP + acol,
                         umma_desc_sw128(doa + kk * 2048, B2_Q * 128, 1024), idesc_acc, (it > 0 || kk > 0) ? 1u : 0u);
          umma_bf16_ts_u(leader, tmem_base + Cfg::TM_DK, tdS + acol,
                         umma_desc_sw128(qa + kk * 2048, B2_Q * 128, 1024), idesc_acc, (it > 0 || kk > 0) ? 1u : 0u);
        }
        // dQ^T = K^T dS^T (K = 128 kv rows -> 8 steps), over the dP^T buffer of this step (after dK above)
#pragma unroll
        for (int kk = 0; kk < B2_KV / 16; ++kk)
          umma_bf16_ss_u(leader, tdS, umma_desc_sw128(ka + kk * 2048, K_LBO, 1024),
                         umma_desc_sw128(dsa + kk * 2048, B2_KV * 128, 1024), idesc_dq, kk > 0 ? 1u : 0u);
        umma_commit_u(leader, &dq_full[pb]);
        umma_commit_u(leader, &q_empty[st]);
        umma_commit_u(leader, &pds_empty[pb]);
      };
      // Two queues, polled in turn: S^T / dP^T of step s_next (needs its Q / dO stage, and its TMEM buffer free:
      // the scores of step s_next - 2 loaded into registers and dQ^T of step s_next - 2 drained) and the gradient
      // products of step g_next (needs P^T / dS^T in shared memory). The scores may run two steps ahead.
      int s_next = 0, g_next = 0;
      uint32_t idle = 0;
      while (ok && g_next < n_iter) {
        bool progressed = false;
        // every lane probes; the vote makes the decision the same in all lanes
        if (s_next < n_iter &&
            __all_sync(0xffffffffu, mbar_test_wait(&q_full[s_next % B2_QST], (s_next / B2_QST) & 1) &&
                                        mbar_test_wait(&s_empty[s_next & 1], ((s_next >> 1) & 1) ^ 1) &&
                                        mbar_test_wait(&dq_empty[s_next & 1], ((s_next >> 1) & 1) ^ 1))) {
          issue_s(s_next);
          ++s_next;
          progressed = true;
        }
        if (g_next < s_next && __all_sync(0xffffffffu, mbar_test_wait(&pds_full[g_next & 1], (g_next >> 1) & 1))) {
          issue_grads(g_next);
          ++g_next;
          progressed = true;
        }
        if (progressed) {
          idle = 0;
        } else if (++idle > GF_WAIT_LIMIT) {
          if (p.status && leader) atomicCAS(p.status, 0, GF_ERR_WAIT_SOFTMAX);
          ok = false;
        } else if (idle > 64) {
          __nanosleep(32);
        }
      }
      if (ok) umma_commit_u(leader, acc_full);
    }
  } else if (warp >= 12) {
    // ---------------------------------------------------------------- dQ drain warps (12..15)
    // Warp w owns TMEM lanes 32 * (w % 4) .. +31 = head-dim rows of dQ^T, 64 query columns per thread. Half a
    // tile at a time goes to shared memory as [32 query rows][HD] (a warp stores 32 consecutive floats, no bank
    // conflicts) and from there to the accumulator as one bulk add-reduction.
    const int lane_grp = warp & 3;
    const int d = lane_grp * 32 + lane;
    const uint32_t tlane = (uint32_t)(lane_grp * 32) << 16;
    float* stage = reinterpret_cast<float*>(smem + Cfg::OFF_DQS);
    const bool issuer = (warp == 12 && lane == 0);
    const long long tiles_per_head = p.S / B2_Q;
    for (int it = 0; it < n_iter; ++it) {
      const int st = it & 1;
      // The four warps meet at named barriers below, so they must agree on giving up: the outcome of the
      // bounded wait is AND-reduced over the warpgroup (itself a barrier that every warp reaches).
      uint32_t all_ok;
      {
        const uint32_t mine = mbar_wait(&dq_full[st], (it >> 1) & 1) ? 1u : 0u;
        asm volatile(
            "{\n\t.reg .pred p, q;\n\t"
            "setp.ne.u32 p, %1, 0;\n\t"
            "bar.red.and.pred q, 1, 128, p;\n\t"
            "selp.u32 %0, 1, 0, q;\n\t}\n"
            : "=r"(all_ok)
            : "r"(mine)
            : "memory");
      }
      if (!all_ok) {
        if (p.status) atomicCAS(p.status, 0, GF_ERR_WAIT_TMEM_FULL);
        break;
      }
      tc_fence_after();
      const int h = hk * G + it / per_head;
      const int i = i_start + it % per_head;
      uint32_t rq[2][32];
      tmem_ld32(tmem_base + st * 128 + Cfg::TM_DP + tlane, rq[0]);
      tmem_ld32(tmem_base + st * 128 + Cfg::TM_DP + 32 + tlane, rq[1]);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&dq_empty[st]);
      float* tile = p.dq_acc + (((long long)b * p.Hq + h) * tiles_per_head + i) * (B2_Q * HD);
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        // the previous reduction has read the staging buffer
        if (issuer) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (d < HD) {
#pragma unroll
          for (int e = 0; e < 32; ++e) stage[e * HD + d] = __uint_as_float(rq[half][e]);
        }
        fence_proxy_async_smem();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (issuer) {
          asm volatile("cp.reduce.async.bulk.global.shared::cta.bulk_group.add.f32 [%0], [%1], %2;" ::"l"(
                           tile + half * (B2_Q / 2) * HD),
                       "r"(smem_u32(stage)), "r"((uint32_t)Cfg::DQ_HALF_BYTES)
                       : "memory");
          asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        }
      }
    }
    // the reductions must have left shared memory (and be performed) before the CTA exits
    if (issuer) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
  } else if (warp >= 4) {
    // ---------------------------------------------------------------- compute warps (4..11)
    // Warps 4..7 own query columns 0..31 of S^T / dP^T, warps 8..11 columns 32..63; within a group, warp w owns
    // TMEM lanes 32 * (w % 4) .. +31, one kv row per thread.
    const int hf = (warp >> 2) - 1;
    const int lane_grp = warp & 3;
    const int r = lane_grp * 32 + lane;
    const int kv_idx = j * B2_KV + r;
    const uint32_t tlane = (uint32_t)(lane_grp * 32) << 16;
    const float sl2 = p.scale * 1.4426950408889634f;
    bool ok = true;

    for (int it = 0; it < n_iter && ok; ++it) {
      const int st = it % B2_QST, pb = it & 1;
      const int i = i_start + it % per_head;
      if (!mbar_wait_warp(&s_full[pb], (it >> 1) & 1)) {
        if (p.status) atomicCAS(p.status, 0, GF_ERR_WAIT_TMEM_FULL);
        ok = false;
        break;
      }
      tc_fence_after();
      uint32_t sv[32], dpv[32];
      tmem_ld32(tmem_base + pb * 128 + Cfg::TM_S + hf * 32 + tlane, sv);
      tmem_ld32(tmem_base + pb * 128 + Cfg::TM_DP + hf * 32 + tlane, dpv);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s_empty[pb]);
      const float4* nl4 = reinterpret_cast<const float4*>(sStat + st * 2 * B2_Q + hf * 32);
      const float4* de4 = reinterpret_cast<const float4*>(sStat + st * 2 * B2_Q + B2_Q + hf * 32);
      const int q0 = i * B2_Q + hf * 32;
      const bool diag = p.causal && (q0 < j * B2_KV + B2_KV);  // these columns touch the diagonal
      uint32_t pp[16], dd[16];
#pragma unroll
      for (int e4 = 0; e4 < 8; ++e4) {
        const float4 nl = nl4[e4], de = de4[e4];
        const float nls[4] = {nl.x, nl.y, nl.z, nl.w};
        const float des[4] = {de.x, de.y, de.z, de.w};
        float pv[4], dv[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int e = e4 * 4 + u;
          float pe = ex2_approx(fmaf(__uint_as_float(sv[e]), sl2, nls[u]));
          if (diag && q0 + e < kv_idx) pe = 0.f;
          pv[u] = pe;
          dv[u] = pe * (__uint_as_float(dpv[e]) - des[u]);
        }
        pp[e4 * 2] = pack_bf16x2(pv[0], pv[1]);
        pp[e4 * 2 + 1] = pack_bf16x2(pv[2], pv[3]);
        dd[e4 * 2] = pack_bf16x2(dv[0], dv[1]);
        dd[e4 * 2 + 1] = pack_bf16x2(dv[2], dv[3]);
      }
      // P^T and dS^T over the first 16 columns of this warp's own S^T / dP^T columns (already in registers)
      tmem_st16(tmem_base + pb * 128 + Cfg::TM_S + hf * 32 + tlane, pp);
      tmem_st16(tmem_base + pb * 128 + Cfg::TM_DP + hf * 32 + tlane, dd);
      if (!mbar_wait_warp(&pds_empty[pb], ((it >> 1) & 1) ^ 1)) {
        if (p.status) atomicCAS(p.status, 0, GF_ERR_WAIT_SOFTMAX);
        ok = false;
        break;
      }
      uint8_t* sDSb = sDS + pb * Cfg::PT_BYTES;
#pragma unroll
      for (int c4 = 0; c4 < 4; ++c4) {
        const uint32_t off = sw128_offset((uint32_t)r, (uint32_t)(hf * 4 + c4));
        *reinterpret_cast<uint4*>(sDSb + off) = make_uint4(dd[c4 * 4], dd[c4 * 4 + 1], dd[c4 * 4 + 2], dd[c4 * 4 + 3]);
      }
      tmem_st_wait();
      tc_fence_before();
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(&pds_full[pb]);
    }
    if (ok) {
      if (!mbar_wait_warp(acc_full, 0)) {
        if (p.status) atomicCAS(p.status, 0, GF_ERR_WAIT_TMEM_FULL);
      } else {
        tc_fence_after();
        __nv_bfloat16* dkr = p.dK + (long long)(row_base + kv_idx) * p.lddk + hk * HD;
        __nv_bfloat16* dvr = p.dV + (long long)(row_base + kv_idx) * p.lddv + hk * HD;
        // each group writes half of the head dimension; dK gets the softmax scale here
#pragma unroll
        for (int cc = 0; cc < HD / 64; ++cc) {
          const int c = hf * (HD / 64) + cc;
          uint32_t rk[32], rv[32];
          if (n_iter > 0) {
            tmem_ld32(tmem_base + Cfg::TM_DK + c * 32 + tlane, rk);
            tmem_ld32(tmem_base + Cfg::TM_DV + c * 32 + tlane, rv);
            tmem_ld_wait();
          } else {
#pragma unroll
            for (int e = 0; e < 32; ++e) rk[e] = rv[e] = 0u;
          }
          if (kv_idx < p.S) {
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4) {
              uint4 uk, uv;
              uint32_t* pk = reinterpret_cast<uint32_t*>(&uk);
              uint32_t* pv = reinterpret_cast<uint32_t*>(&uv);
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const int idx = q4 * 8 + e * 2;
                pk[e] = pack_bf16x2(__uint_as_float(rk[idx]) * p.scale, __uint_as_float(rk[idx + 1]) * p.scale);
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

// delta[b,h,s] = sum_d O * dO and nlse2 = -lse * log2(e); one warp per (token, head).
__global__ void attn_bwd_prep2_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ dout,
                                      const float* __restrict__ lse, float* __restrict__ delta,
                                      float* __restrict__ nlse2, int B, int S, int Hq, int HD, long long ldo,
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
  for (int d = lane * 4; d < HD; d += 128) {
    const uint2 a = *reinterpret_cast<const uint2*>(op + d);
    const uint2 g = *reinterpret_cast<const uint2*>(dp + d);
    const float2 a0 = unpack_bf16x2(a.x), a1 = unpack_bf16x2(a.y), g0 = unpack_bf16x2(g.x), g1 = unpack_bf16x2(g.y);
    acc += a0.x * g0.x + a0.y * g0.y + a1.x * g1.x + a1.y * g1.y;
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
  if (lane == 0) {
    const long long bb = t / S, s = t % S;
    const long long idx = (bb * Hq + h) * S + s;
    delta[idx] = acc;
    nlse2[idx] = -lse[idx] * 1.4426950408889634f;
  }
}

// dq[(b * S + i * 64 + q), h * HD + d] = bf16(scale * acc[b][h][i][q][d]); one thread per four head-dim elements.
__global__ void dq_tiles_to_bf16_kernel(const float* __restrict__ acc, __nv_bfloat16* __restrict__ dq, int B, int S,
                                        int Hq, int HD, long long lddq, float scale) {
  const int vpr = HD >> 2;
  const long long total = (long long)B * Hq * S * vpr;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const int v = (int)(idx % vpr);
    long long t = idx / vpr;          // (b, h, s)
    const int sidx = (int)(t % S);
    t /= S;
    const int h = (int)(t % Hq);
    const long long bb = t / Hq;
    const float4 f = *reinterpret_cast<const float4*>(acc + idx * 4);
    uint2 o;
    o.x = pack_bf16x2(f.x * scale, f.y * scale);
    o.y = pack_bf16x2(f.z * scale, f.w * scale);
    *reinterpret_cast<uint2*>(dq + (bb * S + sidx) * lddq + (long long)h * HD + v * 4) = o;
  }
}

template <int HD>
static int launch_fa_bwd2(const void* q, const void* k, const void* v, const void* dout, long long ldq, long long ldk,
                          long long ldv, long long lddo, FaBwd2Params& p, cudaStream_t stream) {
  using Cfg = FaBwd2Cfg<HD>;
  static gf::DeviceOnce configured;
  auto kern = fa_bwd2_kernel<HD>;
  if (configured.todo()) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES) != cudaSuccess)
      return GFH_CUDA;
    configured.mark();
  }
  const uint64_t T = (uint64_t)p.B * p.S;
  CUtensorMap tq, tk, tv, tdo;
  int rc = make_tmap_2d(&tq, q, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, T, (uint64_t)p.Hq * HD, ldq * 2, B2_Q, 64);
  if (rc) return rc;
  rc = make_tmap_2d(&tdo, dout, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, T, (uint64_t)p.Hq * HD, lddo * 2, B2_Q, 64);
  if (rc) return rc;
  rc = make_tmap_2d(&tk, k, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, T, (uint64_t)p.Hkv * HD, ldk * 2, B2_KV, 64);
  if (rc) return rc;
  rc = make_tmap_2d(&tv, v, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, T, (uint64_t)p.Hkv * HD, ldv * 2, B2_KV, 64);
  if (rc) return rc;
  dim3 grid(p.Hkv, p.S / B2_KV, p.B);
  kern<<<grid, B2_THREADS, Cfg::SMEM_BYTES, stream>>>(tq, tk, tv, tdo, p);
  return cudaGetLastError() == cudaSuccess ? GFH_OK : GFH_CUDA;
}

}  // namespace gf

using namespace gf;

// delta and nlse2 are fp32 [B, Hq, S]; dq_acc (fp32 [B*S, Hq*HD]) is zeroed when given.
GF_API int gf_attn_bwd_prep2(const void* o, const void* dout, const float* lse, float* delta, float* nlse2,
                             float* dq_acc, int B, int S, int Hq, int HD, long long ldo, long long lddo,
                             void* stream) {
  gf::enter();
  if ((HD % 4) || (ldo % 4) || (lddo % 4)) return GFH_BAD_ARG;
  const long long warps = (long long)B * S * Hq;
  const int threads = 256;
  const long long blocks = (warps * 32 + threads - 1) / threads;
  attn_bwd_prep2_kernel<<<(unsigned)blocks, threads, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)o, (const __nv_bfloat16*)dout, lse, delta, nlse2, B, S, Hq, HD, ldo, lddo);
  if (dq_acc) cudaMemsetAsync(dq_acc, 0, (size_t)B * S * Hq * HD * sizeof(float), (cudaStream_t)stream);
  return cudaGetLastError() == cudaSuccess ? GFH_OK : GFH_CUDA;
}

// dq_acc: fp32 [B, Hq, S / 64, 64, HD] zero-initialised (gf_attn_bwd_prep2 does it); it receives dQ / scale, so
// convert afterwards with gf_dq_tiles_to_bf16(..., scale). S must be a multiple of 128.
GF_API int gf_flash_attn_bwd2(const void* q, const void* k, const void* v, const void* dout, const float* nlse2,
                              const float* delta, float* dq_acc, void* dk, void* dv, int B, int S, int Hq, int Hkv,
                              int head_dim, long long ldq, long long ldk, long long ldv, long long lddo,
                              long long lddk, long long lddv, float scale, int causal, int* status, void* stream) {
  gf::enter();
  if (B <= 0 || S <= 0 || (S % B2_KV) || Hq % Hkv) return GFH_BAD_ARG;
  if ((ldq % 8) || (ldk % 8) || (ldv % 8) || (lddo % 8) || (lddk % 8) || (lddv % 8)) return GFH_BAD_ARG;
  FaBwd2Params p;
  p.B = B; p.S = S; p.Hq = Hq; p.Hkv = Hkv; p.causal = causal; p.scale = scale;
  p.nlse2 = nlse2; p.delta = delta; p.dq_acc = dq_acc;
  p.dK = (__nv_bfloat16*)dk; p.lddk = lddk; p.dV = (__nv_bfloat16*)dv; p.lddv = lddv; p.status = status;
  p.head_group = attention_head_group(Hkv);
  if (head_dim == 128) return launch_fa_bwd2<128>(q, k, v, dout, ldq, ldk, ldv, lddo, p, (cudaStream_t)stream);
  if (head_dim == 64) return launch_fa_bwd2<64>(q, k, v, dout, ldq, ldk, ldv, lddo, p, (cudaStream_t)stream);
  return GFH_BAD_ARG;
}

// Converts the tiled fp32 dQ accumulator of gf_flash_attn_bwd2 into bf16 rows with pitch lddq.
GF_API int gf_dq_tiles_to_bf16(const float* acc, void* dq, int B, int S, int Hq, int HD, long long lddq, float scale,
                               void* stream) {
  gf::enter();
  if ((HD % 4) || (lddq % 4) || (S % B2_Q)) return GFH_BAD_ARG;
  const long long total = (long long)B * Hq * S * (HD / 4);
  long long g = (total + 255) / 256;
  const long long cap = (long long)sm_count() * 16;
  if (g > cap) g = cap;
  if (g < 1) g = 1;
  dq_tiles_to_bf16_kernel<<<(unsigned)g, 256, 0, (cudaStream_t)stream>>>(acc, (__nv_bfloat16*)dq, B, S, Hq, HD, lddq,
                                                                        scale);
  return cudaGetLastError() == cudaSuccess ? GFH_OK : GFH_CUDA;
}

