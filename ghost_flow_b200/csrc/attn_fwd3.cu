// FlashAttention forward, third generation. Same tiling as attn_fwd2.cu (one CTA owns 256 query rows of one
// head as two 128-row tiles, each with its own four softmax warps), with the two changes that keep the tensor
// pipe busy while the softmax warps work:
//
//  * The probabilities never touch shared memory. A softmax thread reads its row of S = Q K^T from tensor
//    memory, and writes P = exp2(...) as packed bf16 back into the first 64 columns of the same S region
//    (tcgen05.st); O += P V then takes its A operand from tensor memory. The 64 KB of shared memory that held
//    P now double-buffer K.
//  * The MMA warp issues  P V (tile t, step j)  followed at once by  Q K^T (tile t, step j + 1)  and only then
//    turns to the other tile. While the softmax warps of one tile are busy, the tensor pipe runs the two
//    products of the other tile, so in steady state the tiles alternate instead of both waiting for both
//    softmaxes. MMAs execute in issue order, so the Q K^T that overwrites S (and with it P) starts after the
//    P V that read it, and the commit that announces the new S also covers that P V: a softmax thread that
//    sees S(j + 1) may rescale O without a further wait.
//
// The output accumulates in TMEM across KV tiles and is rescaled in place only when a row maximum has grown by
// more than 2^8 since the last rescale; P is exp2 against that (possibly stale) reference maximum.
//
// Replaces ghostflow-cuda/src/optimized_kernels.cu:185-248 and the CPU algorithm of
// ghostflow-nn/src/flash_attention.rs:122-250.
#include "gf_host.h"
#include "gf_ptx.cuh"

namespace gf {

constexpr int F3_TILE = 128;      // query rows per tile, kv rows per step
constexpr int F3_THREADS = 384;   // warpgroup 0: TMA warp, MMA warp, two idle warps; warpgroups 1 and 2: softmax of tile 0 / 1
// Registers move from warpgroup 0 to the softmax warpgroups (a softmax thread keeps its whole row of 128
// scores in registers): 128 x 64 + 256 x 216 = 63488 of the 65536 registers of an SM.
constexpr int F3_REGS_CTRL = 64;
constexpr int F3_REGS_SOFTMAX = 216;
constexpr float F3_RESCALE_THRESHOLD = 8.0f;  // log2 units

struct Fa3Params {
  int B, S, Hq, Hkv;
  int causal;
  float scale;
  __nv_bfloat16* O;
  long long ldo;
  float* lse;
  int* status;
  int head_group;   // heads whose CTAs are dispatched together (see the kernel's block decoding)
};

template <int HD>
struct Fa3Cfg {
  static constexpr int CH = HD / 64;
  static constexpr int TILE_BYTES = F3_TILE * HD * 2;      // one Q / K / V tile
  static constexpr int KV_STAGES = 2;
  static constexpr int OFF_Q = 0;                                   // 2 tiles
  static constexpr int OFF_K = OFF_Q + 2 * TILE_BYTES;              // KV_STAGES stages
  static constexpr int OFF_V = OFF_K + KV_STAGES * TILE_BYTES;      // KV_STAGES stages
  static constexpr int OFF_BAR = OFF_V + KV_STAGES * TILE_BYTES;
  static constexpr int SMEM_BYTES = OFF_BAR + 256 + 1024;
  static constexpr int TM_S = 0;      // + t * 128; P (bf16 pairs) occupies the first 64 columns of the same region
  static constexpr int TM_O = 256;    // + t * 128
  static constexpr int TMEM_COLS = 512;
};

template <int HD>
__global__ void __launch_bounds__(F3_THREADS, 1)
fa_fwd3_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
               const __grid_constant__ CUtensorMap tmV, const Fa3Params p) {
  using Cfg = Fa3Cfg<HD>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem + Cfg::OFF_Q;
  uint8_t* sK = smem + Cfg::OFF_K;
  uint8_t* sV = smem + Cfg::OFF_V;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::OFF_BAR);
  uint64_t* q_full = bars + 0;
  uint64_t* k_full = bars + 1;    // [2]
  uint64_t* k_empty = bars + 3;   // [2]
  uint64_t* v_full = bars + 5;    // [2]
  uint64_t* v_empty = bars + 7;   // [2]
  uint64_t* s_full = bars + 9;    // [2] per tile
  uint64_t* p_full = bars + 11;   // [2] per tile
  uint64_t* o_done = bars + 13;   // [2] per tile
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 15);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_qb = (p.S + 2 * F3_TILE - 1) / (2 * F3_TILE);
  // CTAs are dispatched in linear block order. Heads are taken in groups of head_group: inside a group the heaviest
  // query block (most KV tiles under a causal mask) of every head comes first, then the next block, so long CTAs
  // start first and short ones fill the tail, while the CTAs in flight at any time belong to few heads, whose K / V
  // (re-read by every query block) stay in L2.
  int qb, h;
  {
    const int H = gridDim.x, NT = gridDim.y;
    const int lin = blockIdx.x + H * blockIdx.y;
    const int gs = p.head_group;
    const int g = lin / (gs * NT);
    const int rem = lin - g * gs * NT;
    const int gs_g = min(gs, H - g * gs);
    qb = n_qb - 1 - rem / gs_g;
    h = g * gs + rem % gs_g;
  }
  const int b = blockIdx.z;
  const int hk = h / (p.Hq / p.Hkv);
  const int n_kv_all = (p.S + F3_TILE - 1) / F3_TILE;
  const int row_base = b * p.S;
  int n_kv[2];
#pragma unroll
  for (int t = 0; t < 2; ++t) {
    const int q0 = qb * 2 * F3_TILE + t * F3_TILE;
    if (q0 >= p.S) n_kv[t] = 0;
    else n_kv[t] = p.causal ? min(q0 / F3_TILE + 1, n_kv_all) : n_kv_all;
  }
  const int n_j = max(n_kv[0], n_kv[1]);

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&p_full[i], 4);
      mbar_init(&o_done[i], 1);
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

  if (warp < 4) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(F3_REGS_CTRL));
  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      mbar_expect_tx(q_full, 2 * Cfg::TILE_BYTES);
#pragma unroll
      for (int t = 0; t < 2; ++t)
#pragma unroll
        for (int c = 0; c < Cfg::CH; ++c)
          tma_load_2d(sQ + t * Cfg::TILE_BYTES + c * (F3_TILE * 128), &tmQ, q_full, h * HD + c * 64,
                      row_base + qb * 2 * F3_TILE + t * F3_TILE);
      for (int j = 0; j < n_j; ++j) {
        const int st = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!mbar_wait(&k_empty[st], ph ^ 1)) {
          if (p.status) atomicCAS(p.status, 0, GF_ERR_WAIT_EMPTY);
          break;
        }
        mbar_expect_tx(&k_full[st], Cfg::TILE_BYTES);
#pragma unroll
        for (int c = 0; c < Cfg::CH; ++c)
          tma_load_2d(sK + st * Cfg::TILE_BYTES + c * (F3_TILE * 128), &tmK, &k_full[st], hk * HD + c * 64,
                      row_base + j * F3_TILE);
        if (!mbar_wait(&v_empty[st], ph ^ 1)) {
          if (p.status) atomicCAS(p.status, 0, GF_ERR_WAIT_EMPTY);
          break;
        }
        mbar_expect_tx(&v_full[st], Cfg::TILE_BYTES);
#pragma unroll
        for (int c = 0; c < Cfg::CH; ++c)
          tma_load_2d(sV + st * Cfg::TILE_BYTES + c * (F3_TILE * 128), &tmV, &v_full[st], hk * HD + c * 64,
                      row_base + j * F3_TILE);
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_qk = umma_idesc_bf16(F3_TILE, F3_TILE, 0, 0);
      constexpr uint32_t idesc_pv = umma_idesc_bf16(F3_TILE, HD, 0, 1);
      bool ok = mbar_wait(q_full, 0);
      if (!ok && p.status) atomicCAS(p.status, 0, GF_ERR_WAIT_FULL);
      // S_t = Q_t K(j)^T, announced on s_full[t]
      auto issue_qk = [&](int t, int j) {
        const uint32_t qa = smem_u32(sQ + t * Cfg::TILE_BYTES);
        const uint32_t ka = smem_u32(sK + (j & 1) * Cfg::TILE_BYTES);
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint32_t off = (kk >> 2) * (F3_TILE * 128) + (kk & 3) * 32;
          umma_bf16_ss(tmem_base + Cfg::TM_S + t * 128, umma_desc_sw128(qa + off, 16, 1024),
                       umma_desc_sw128(ka + off, 16, 1024), idesc_qk, kk > 0 ? 1u : 0u);
        }
        umma_commit(&s_full[t]);
      };
      if (ok && n_j > 0) {
        if (!mbar_wait(&k_full[0], 0)) {
          if (p.status) atomicCAS(p.status, 0, GF_ERR_WAIT_FULL);
          ok = false;
        } else {
          tc_fence_after();
#pragma unroll
          for (int t = 0; t < 2; ++t)
            if (n_kv[t] > 0) issue_qk(t, 0);
          umma_commit(&k_empty[0]);
        }
      }
      for (int j = 0; j < n_j && ok; ++j) {
        const int st = j & 1;
        const bool has_next = j + 1 < n_j;
        if (!mbar_wait(&v_full[st], (j >> 1) & 1) ||
            (has_next && !mbar_wait(&k_full[(j + 1) & 1], ((j + 1) >> 1) & 1))) {
          if (p.status) atomicCAS(p.status, 0, GF_ERR_WAIT_FULL);
          ok = false;
          break;
        }
        const uint32_t va = smem_u32(sV + st * Cfg::TILE_BYTES);
#pragma unroll
        for (int t = 0; t < 2; ++t) {
          if (j < n_kv[t]) {
            if (!mbar_wait(&p_full[t], j & 1)) {
              if (p.status) atomicCAS(p.status, 0, GF_ERR_WAIT_SOFTMAX);
              ok = false;
              break;
            }
            tc_fence_after();
            // O_t += P_t V(j): A = P_t from tensor memory (8 columns per 16 kv rows), B = V(j) MN-major
#pragma unroll
            for (int kk = 0; kk < F3_TILE / 16; ++kk)
              umma_bf16_ts(tmem_base + Cfg::TM_O + t * 128, tmem_base + Cfg::TM_S + t * 128 + kk * 8,
                           umma_desc_sw128(va + kk * 2048, F3_TILE * 128, 1024), idesc_pv,
                           (j > 0 || kk > 0) ? 1u : 0u);
            if (j == n_kv[t] - 1) umma_commit(&o_done[t]);
          }
          if (j + 1 < n_kv[t]) issue_qk(t, j + 1);
        }
        if (!ok) break;
        umma_commit(&v_empty[st]);
        if (has_next) umma_commit(&k_empty[(j + 1) & 1]);
      }
    }
  }
  } else {
    // ---------------------------------------------------------------- softmax warps: tile t = warp / 4 - 1
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(F3_REGS_SOFTMAX));
    const int t = (warp >> 2) - 1;
    const int lane_grp = warp & 3;
    const int r = lane_grp * 32 + lane;
    const int q_idx = qb * 2 * F3_TILE + t * F3_TILE + r;
    const uint32_t tlane = (uint32_t)(lane_grp * 32) << 16;
    const uint32_t ts = tmem_base + Cfg::TM_S + t * 128 + tlane;
    const uint32_t to = tmem_base + Cfg::TM_O + t * 128 + tlane;
    const float sl2 = p.scale * 1.4426950408889634f;
    float m_ref = -INFINITY, l = 0.f;
    bool ok = true;
    const int my_n = t ? n_kv[1] : n_kv[0];
    for (int j = 0; j < my_n && ok; ++j) {
      if (!mbar_wait_warp(&s_full[t], j & 1)) {
        if (p.status) atomicCAS(p.status, 0, GF_ERR_WAIT_TMEM_FULL);
        ok = false;
        break;
      }
      tc_fence_after();
      const int kv0 = j * F3_TILE;
      const bool need_mask = (p.causal && (kv0 + F3_TILE - 1 > qb * 2 * F3_TILE + t * F3_TILE)) ||
                             (kv0 + F3_TILE > p.S);
      // ---- the whole row of raw scores into registers
      uint32_t sv[F3_TILE];
#pragma unroll
      for (int c = 0; c < F3_TILE / 32; ++c) tmem_ld32(ts + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&sv[c * 32]));
      tmem_ld_wait();
      if (need_mask) {
#pragma unroll
        for (int i = 0; i < F3_TILE; ++i) {
          const int kv = kv0 + i;
          if (kv >= p.S || (p.causal && kv > q_idx)) sv[i] = 0xff800000u;  // -inf
        }
      }
      // four independent chains: a single running maximum would serialise 64 dependent instructions
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int i = 0; i < F3_TILE; i += 8) {
#pragma unroll
        for (int e = 0; e < 4; ++e)
          mx4[e] = fmaxf(mx4[e], fmaxf(__uint_as_float(sv[i + 2 * e]), __uint_as_float(sv[i + 2 * e + 1])));
      }
      const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      // ---- reference maximum: move it (and rescale O, l) only when the row maximum grew a lot. The commit
      // behind s_full also covered P V (j - 1), so O is quiescent here.
      if (j == 0) {
        m_ref = mx;
      } else {
        const bool grow = (mx - m_ref) * sl2 > F3_RESCALE_THRESHOLD;
        if (__any_sync(0xffffffffu, grow)) {
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
          l *= alpha;
          if (grow) m_ref = mx;
        }
      }
      const float mref_use = (m_ref == -INFINITY) ? 0.f : m_ref;  // row with no visible key yet
      const float mneg = -mref_use * sl2;
      // ---- P = 2^(s*scale*log2e - m_ref*scale*log2e) as bf16 pairs into columns [0, 64) of the S region
      float rs0 = 0.f, rs1 = 0.f;
#pragma unroll
      for (int c = 0; c < F3_TILE / 32; ++c) {
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          const float p0 = ex2_approx(fmaf(__uint_as_float(sv[c * 32 + i]), sl2, mneg));
          const float p1 = ex2_approx(fmaf(__uint_as_float(sv[c * 32 + i + 1]), sl2, mneg));
          rs0 += p0;
          rs1 += p1;
          pk[i >> 1] = pack_bf16x2(p0, p1);
        }
        tmem_st16(ts + c * 16, pk);
      }
      l += rs0 + rs1;
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[t]);
    }
    // ---- epilogue: O / l
    if (ok && my_n > 0) {
      if (!mbar_wait_warp(&o_done[t], 0)) {
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
static int launch_fa3(const void* q, const void* k, const void* v, long long ldq, long long ldk, long long ldv,
                      Fa3Params& p, cudaStream_t stream) {
  using Cfg = Fa3Cfg<HD>;
  static gf::DeviceOnce configured;
  auto kern = fa_fwd3_kernel<HD>;
  if (configured.todo()) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES) != cudaSuccess)
      return GFH_CUDA;
    configured.mark();
  }
  const uint64_t T = (uint64_t)p.B * p.S;
  CUtensorMap tq, tk, tv;
  int rc = make_tmap_2d(&tq, q, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, T, (uint64_t)p.Hq * HD, ldq * 2, F3_TILE, 64);
  if (rc) return rc;
  rc = make_tmap_2d(&tk, k, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, T, (uint64_t)p.Hkv * HD, ldk * 2, F3_TILE, 64);
  if (rc) return rc;
  rc = make_tmap_2d(&tv, v, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, T, (uint64_t)p.Hkv * HD, ldv * 2, F3_TILE, 64);
  if (rc) return rc;
  dim3 grid(p.Hq, (p.S + 2 * F3_TILE - 1) / (2 * F3_TILE), p.B);
  kern<<<grid, F3_THREADS, Cfg::SMEM_BYTES, stream>>>(tq, tk, tv, p);
  return cudaGetLastError() == cudaSuccess ? GFH_OK : GFH_CUDA;
}

}  // namespace gf

// Same contract as gf_flash_attn_fwd (attn_fwd.cu).
GF_API int gf_flash_attn_fwd3(const void* q, const void* k, const void* v, void* o, float* lse, int B, int S, int Hq,
                              int Hkv, int head_dim, long long ldq, long long ldk, long long ldv, long long ldo,
                              float scale, int causal, int* status, void* stream) {
  using namespace gf;
  enter();
  if (B <= 0 || S <= 0 || Hq <= 0 || Hkv <= 0 || Hq % Hkv) return GFH_BAD_ARG;
  if ((ldq % 8) || (ldk % 8) || (ldv % 8) || (ldo % 8)) return GFH_BAD_ARG;
  Fa3Params p;
  p.B = B; p.S = S; p.Hq = Hq; p.Hkv = Hkv; p.causal = causal; p.scale = scale;
  p.O = (__nv_bfloat16*)o; p.ldo = ldo; p.lse = lse; p.status = status;
  p.head_group = attention_head_group(Hq);
  if (head_dim == 128) return launch_fa3<128>(q, k, v, ldq, ldk, ldv, p, (cudaStream_t)stream);
  if (head_dim == 64) return launch_fa3<64>(q, k, v, ldq, ldk, ldv, p, (cudaStream_t)stream);
  return GFH_BAD_ARG;
}
