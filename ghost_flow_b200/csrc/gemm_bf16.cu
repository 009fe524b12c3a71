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
  // Fused all-gather (optional). The first g_copy_ctas CTAs pull every rank's shard of a flat bf16 buffer
  // into this GPU's memory (own shard first, then rank+1, rank+2, ...) and raise one flag per shard; the compute
  // CTAs walk the tiles in the same order and wait (bounded) only for the shards that hold their tile's rows
  // of the gathered operand, so the GEMM starts on local data while remote shards are still in flight.
  int g_operand;            // -1 none, 0 = the rows of A are gathered, 1 = the rows of B (K-major operands only)
  int g_copy_ctas;
  int g_world, g_rank;
  int g_first_shard;        // copy order: g_first_shard, g_first_shard + 1, ... (mod world)
  const void* g_src[8];     // every rank's shard (peer-mapped)
  __nv_bfloat16* g_dst;     // local gathered buffer: shard r lands at g_dst + r * g_shard_elems
  long long g_shard_elems;  // multiple of 8
  long long g_operand_off;  // element offset of the operand's first row inside the gathered buffer
  long long g_operand_ld;   // row pitch of the gathered operand, elements
  int* g_ready;             // local int[world]: epoch value once shard r is complete
  int* g_counters;          // local int[world], zero before launch (reset by the kernel)
  int g_epoch;
  const int* g_version_pad; // this rank's signal pad: wait pad[g_version_idx + r] >= g_version_val before reading rank r
  int g_version_idx, g_version_val;
  // Fused reduce-scatter (optional, row-parallel linear): every rank holds a partial C; rows are owned in
  // contiguous blocks of rs_rows_per_rank. The epilogue stores each partial tile straight into the OWNER rank's
  // staging buffer over NVLink and bumps the owner's arrival counter for that column block; after its own tiles a
  // CTA turns to the reduce phase: it waits (bounded) until all ranks' partials of a column block have arrived
  // and sums them into the local output shard.
  int rs_world, rs_rank;            // rs_world = 0: off
  __nv_bfloat16* rs_stage[8];       // every rank's staging buffer [world][rows_per_rank][N] (peer-mapped)
  int* rs_counters[8];              // every rank's arrival counters int[tiles_n] (peer-mapped, start at zero)
  int rs_rows_per_rank;
  int rs_call;                      // number of earlier calls that used these counters with the same shape
  __nv_bfloat16* rs_out;            // local output [rows_per_rank, N]
  long long rs_ldo;
  int order_n_fast;         // 1: consecutive tiles share the A row block (used when A is the gathered operand)
  int rs_tma;               // partial tiles leave through shared memory and TMA stores (full NVLink packets)
  int rs_interleave;        // > 0: row blocks per owner; the walk then alternates between owners block by block
  // ---- grouped GEMM over row segments (experts of a mixture-of-experts layer). grp_offsets[e] is the first row
  // of segment e in a row-sorted buffer, every entry a multiple of BM, grp_offsets[experts] the total.
  //  mode 1: C[rows, N] = A[rows, K] x B_e, B_e the e-th matrix of a stacked weight (forward / input gradient)
  //  mode 2: C_e[M, N] = A[rows_e, M]^T x B[rows_e, N], the contraction runs over the rows of segment e (weight
  //          gradient); C is stacked [experts, M, N]
  const int* grp_offsets;
  int grp_experts, grp_mode;
  int grp_b_rows;           // rows of one B_e in the stacked tensor map (mode 1)
  // mode 1 fed by an all-to-all dispatch: rows of segment e that came from rank r are
  // [grp_src_start[e * (grp_world + 1) + r], ...[r + 1]); rank r's rows are complete once grp_arrived[r] >= grp_epoch.
  // A tile waits only for the ranks whose rows it reads.
  const int* grp_src_start;
  const int* grp_arrived;
  int grp_world, grp_epoch;
  // scatter epilogue (all-to-all combine fused into the GEMM): output row r goes to rank sc_ret[r].x, row
  // sc_ret[r].y of that rank's buffer sc_dst[rank] (pitch sc_ld); rows with sc_ret[r].y < 0 are padding. When the
  // last CTA is done it stores sc_epoch into sc_flags[peer][sc_rank] of every rank.
  const int2* sc_ret;
  __nv_bfloat16* sc_dst[8];
  int* sc_flags[8];
  long long sc_ld;
  int sc_world, sc_rank, sc_epoch;
  int* sc_counter;
  // split-K for skinny problems (few output tiles, long K): tile index = (k slice, tile); every slice adds its
  // partial product into the fp32 workspace `ws` [M, N] with atomics; a second kernel converts.
  int split_k;
  float* ws;
  int act;                  // epilogue activation after bias and residual: 0 none, 1 ReLU
  int group_m;              // > 0: plain GEMM walks bands of group_m row blocks (keeps a wave's A and B panels in L2)
  int tile_rot;             // rotation of the slow tile index so that the walk starts in the local shard
  // Implicit convolution (stride 1, odd window, "same" padding) over a channels-last image whose rows and images
  // are separated by `pad` zero pixels: pixel (n, y, x) is row (n * Hp + y) * conv_pitch + x of a [rows, C] matrix
  // and the neighbour (y + dy, x + dx) is row + dy * conv_pitch + dx, so the A tile of window tap (ky, kx) is the
  // same 2-D tensor map read `(ky - pad) * conv_pitch + (kx - pad)` rows further on. k block kb covers channels
  // (kb % conv_cpb) * 64 ... of tap kb / conv_cpb. conv_cpb = 0: off.
  int conv_cpb, conv_kw, conv_pitch, conv_pad;
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

// Fused reduce-scatter: every epilogue warp stages 32 rows x 128 columns of a partial tile in shared memory and
// sends them to the owner rank with one TMA store, so NVLink carries full packets instead of 16-byte stores.
constexpr int RS_STAGE_COLS = 128;
constexpr int RS_STAGE_BYTES = 4 * 32 * RS_STAGE_COLS * 2;
struct RsMaps {
  CUtensorMap m[8];         // every rank's staging buffer [world * rows_per_rank, N], box 32 x 128, no swizzle
};

__device__ __forceinline__ void set_status(int* status, int code) {
  if (status) atomicCAS(status, 0, code);
}

// Tile walk: by default consecutive tiles share the B column block (tm fastest); with order_n_fast they share
// the A row block. The slow index is rotated by tile_rot.
__device__ __forceinline__ void tile_coords(const GemmParams& p, int tile, int& tm, int& tn) {
  if (p.group_m > 0) {
    // Bands of group_m row blocks; inside a band the row index runs fastest, so one wave of CTAs touches about
    // group_m A panels and (CTAs / group_m) B panels instead of a whole operand. `s` is the position in the
    // row-block order, which is the identity for a plain GEMM, rotated so that the walk starts in the shard that
    // is local (fused all-gather of A), or alternating between owner ranks, the next rank first and this rank
    // last (fused reduce-scatter: spreads the NVLink stores of the epilogue evenly over the run of the kernel).
    const int per_band = p.group_m * p.tiles_n;
    const int band = tile / per_band;
    const int first = band * p.group_m;
    const int rows = min(p.group_m, p.tiles_m - first);
    const int r = tile - band * per_band;
    const int s = first + r % rows;
    tn = r / rows;
    if (p.rs_interleave > 0) {
      int owner = s % p.rs_world + p.rs_rank + 1;
      if (owner >= p.rs_world) owner -= p.rs_world;
      tm = owner * p.rs_interleave + s / p.rs_world;
    } else {
      tm = s + p.tile_rot;
      if (tm >= p.tiles_m) tm -= p.tiles_m;
    }
  } else if (p.order_n_fast) {
    tn = tile % p.tiles_n;
    tm = tile / p.tiles_n + p.tile_rot;
    if (tm >= p.tiles_m) tm -= p.tiles_m;
  } else {
    tm = tile % p.tiles_m;
    tn = tile / p.tiles_m + p.tile_rot;
    if (tn >= p.tiles_n) tn -= p.tiles_n;
  }
}

struct TileInfo {
  int tm, tn;
  int a_row;        // row (M) coordinate of the A tile in its tensor map
  int b_row;        // row (N) coordinate of the B tile in its tensor map (K-major B)
  int b_k_add;      // added to the k coordinate of an MN-major B (stacked [experts * K, N])
  int k_begin;      // first k of the contraction
  int nkb;          // k blocks of the contraction
  long long c_row_add;  // added to the output row
};

// Fills `t` for tile index `tile`; false if the tile has nothing to compute (grouped modes).
__device__ __forceinline__ bool tile_info(const GemmParams& p, int tile, int num_kb, TileInfo& t) {
  t.b_k_add = 0; t.k_begin = 0; t.nkb = num_kb; t.c_row_add = 0;
  if (p.grp_mode == 2) {
    const int per = p.tiles_m * p.tiles_n;
    const int e = tile / per;
    const int r = tile - e * per;
    t.tm = r % p.tiles_m;
    t.tn = r / p.tiles_m;
    t.a_row = t.tm * BM;
    t.b_row = 0;
    const int k0 = __ldg(p.grp_offsets + e), k1 = __ldg(p.grp_offsets + e + 1);
    t.k_begin = k0;
    t.nkb = (k1 - k0) / BK;
    t.c_row_add = (long long)e * p.M;
    return true;              // an empty segment still owes zeros (or nothing, when accumulating) to the output
  }
  if (p.split_k > 1) {
    const int per = p.tiles_m * p.tiles_n;
    const int ks = tile / per;
    tile_coords(p, tile - ks * per, t.tm, t.tn);
    t.a_row = t.tm * BM;
    t.b_row = 0;
    const int kbs = (num_kb + p.split_k - 1) / p.split_k;
    t.k_begin = ks * kbs * BK;
    t.nkb = min(kbs, num_kb - ks * kbs);
    return t.nkb > 0;
  }
  tile_coords(p, tile, t.tm, t.tn);
  t.a_row = t.tm * BM;
  t.b_row = 0;
  if (p.grp_mode == 1) {
    if (t.a_row >= __ldg(p.grp_offsets + p.grp_experts)) return false;
    int e = 0;
    while (e + 1 < p.grp_experts && __ldg(p.grp_offsets + e + 1) <= t.a_row) ++e;
    t.b_row = e * p.grp_b_rows;
    t.b_k_add = e * p.grp_b_rows;
    t.c_row_add = -(long long)(e + 1);      // producer: the segment index, recovered below (outputs add nothing)
  }
  return true;
}

// Copy CTAs of the fused all-gather. One thread per copy CTA drives the bulk-copy engine: peer shard ->
// shared-memory ring (cp.async.bulk, completion on an mbarrier; plain bulk loads, no multicast) -> local gathered
// buffer (cp.async.bulk store). The ring keeps (G_CHUNKS - 2) x 16 KB in flight per CTA without using
// registers or issue slots, so a handful of copy CTAs fills the NVLink ports. Every copy CTA takes a slice of
// each shard, shard by shard in arrival order (own shard first), so the whole copy bandwidth goes to the shard
// the compute CTAs need next.
constexpr int G_CHUNK = 16384;
constexpr int G_CHUNKS = 8;

__device__ __forceinline__ void gather_role(const GemmParams& p, uint8_t* smem) {
  uint64_t* bar = reinterpret_cast<uint64_t*>(smem + G_CHUNKS * G_CHUNK);
  if (threadIdx.x != 0) return;
  for (int i = 0; i < G_CHUNKS; ++i) mbar_init(&bar[i], 1);
  mbar_fence_init();
  const long long shard_bytes = p.g_shard_elems * 2;
  long long per = (shard_bytes + p.g_copy_ctas - 1) / p.g_copy_ctas;
  per = (per + 255) / 256 * 256;
  const long long lo = (long long)blockIdx.x * per;
  long long hi = lo + per;
  if (hi > shard_bytes) hi = shard_bytes;
  const int nchunks = hi > lo ? (int)((hi - lo + G_CHUNK - 1) / G_CHUNK) : 0;
  uint32_t issued = 0;  // chunks loaded so far over all shards: stage = issued % G_CHUNKS, phase = (issued / G_CHUNKS) & 1
  for (int order = 0; order < p.g_world; ++order) {
    int src = p.g_first_shard + order;
    if (src >= p.g_world) src -= p.g_world;
    bool ok = true;
    if (src != p.g_rank && p.g_version_pad) {
      ok = false;
      for (uint32_t it = 0; it < GF_WAIT_LIMIT; ++it) {
        int v;
        asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p.g_version_pad + p.g_version_idx + src) : "memory");
        if (v >= p.g_version_val) { ok = true; break; }
        __nanosleep(100);
      }
      if (!ok) set_status(p.status, GF_ERR_WAIT_PEER);
    }
    if (ok && nchunks > 0) {
      const char* sbase = reinterpret_cast<const char*>(p.g_src[src]) + lo;
      char* dbase = reinterpret_cast<char*>(p.g_dst) + (long long)src * shard_bytes + lo;
      constexpr int LAG = G_CHUNKS - 2;
      const uint32_t first = issued;
      for (int c = 0; c < nchunks + LAG; ++c) {
        if (c < nchunks) {
          // the store that last read this stage must be done with shared memory (all but the newest store group)
          asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
          const uint32_t n = first + c;
          const int st = n % G_CHUNKS;
          const long long off = (long long)c * G_CHUNK;
          const uint32_t bytes = (uint32_t)((hi - lo - off) < G_CHUNK ? (hi - lo - off) : G_CHUNK);
          mbar_expect_tx(&bar[st], bytes);
          asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                       ::"r"(smem_u32(smem + st * G_CHUNK)), "l"(sbase + off), "r"(bytes), "r"(smem_u32(&bar[st]))
                       : "memory");
        }
        const int d = c - LAG;
        if (d >= 0) {
          const uint32_t n = first + d;
          const int st = n % G_CHUNKS;
          if (!mbar_wait(&bar[st], (n / G_CHUNKS) & 1)) {
            set_status(p.status, GF_ERR_WAIT_FULL);
            ok = false;
            break;
          }
          const long long off = (long long)d * G_CHUNK;
          const uint32_t bytes = (uint32_t)((hi - lo - off) < G_CHUNK ? (hi - lo - off) : G_CHUNK);
          asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
                       ::"l"(dbase + off), "r"(smem_u32(smem + st * G_CHUNK)), "r"(bytes)
                       : "memory");
          asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        }
      }
      issued = first + nchunks;
      asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    }
    __threadfence();
    const int prev = atomicAdd(p.g_counters + src, 1);
    if (prev == p.g_copy_ctas - 1) {
      p.g_counters[src] = 0;
      __threadfence();
      if (ok) asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(p.g_ready + src), "r"(p.g_epoch) : "memory");
    }
    if (!ok) {
      error_drain_pause();
      return;
    }
  }
}

template <int BN, bool A_MN, bool B_MN>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const GemmParams p, const __grid_constant__ RsMaps rsm) {
  using Cfg = GemmCfg<BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + Cfg::STAGES * Cfg::STAGE_BYTES);
  uint64_t* empty_bar = full_bar + Cfg::STAGES;
  uint64_t* tfull_bar = empty_bar + Cfg::STAGES;
  uint64_t* tempty_bar = tfull_bar + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
  uint8_t* rs_stage_smem = smem + Cfg::STAGES * Cfg::STAGE_BYTES + 256;    // behind the barriers; only with p.rs_tma

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_kb = (p.K + BK - 1) / BK;
  const int num_tiles = p.tiles_m * p.tiles_n * (p.grp_mode == 2 ? p.grp_experts : 1) * (p.split_k > 1 ? p.split_k : 1);
  const int n_copy = p.g_operand >= 0 ? p.g_copy_ctas : 0;
  if ((int)blockIdx.x < n_copy) {
    gather_role(p, smem);
    return;
  }
  const int cta = (int)blockIdx.x - n_copy;
  const int nctas = (int)gridDim.x - n_copy;

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
      for (int tile = cta; tile < num_tiles && ok; tile += nctas) {
        TileInfo ti;
        if (!tile_info(p, tile, num_kb, ti)) continue;
        const int m0 = ti.a_row, n0 = ti.tn * BN;
        if (p.grp_src_start) {
          const int e = (int)(-ti.c_row_add) - 1;
          const int* ss = p.grp_src_start + e * (p.grp_world + 1);
          for (int r = 0; r < p.grp_world && ok; ++r) {
            if (__ldg(ss + r) >= m0 + BM || __ldg(ss + r + 1) <= m0) continue;
            uint32_t spins = 0;
            while (true) {
              int v;
              asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p.grp_arrived + r) : "memory");
              if (v >= p.grp_epoch) break;
              if (++spins > GF_WAIT_LIMIT) { ok = false; break; }
              __nanosleep(64);
            }
          }
          if (!ok) {
            set_status(p.status, GF_ERR_WAIT_PEER);
            break;
          }
          fence_proxy_async_all();
        }
        if (p.g_operand >= 0) {
          // shards that hold the rows of the gathered operand read by this tile
          const long long r0 = p.g_operand == 0 ? m0 : n0;
          const long long rmax = p.g_operand == 0 ? p.M : p.N;
          long long r1 = r0 + (p.g_operand == 0 ? BM : BN);
          if (r1 > rmax) r1 = rmax;
          const long long e0 = p.g_operand_off + r0 * p.g_operand_ld;
          const long long e1 = p.g_operand_off + (r1 - 1) * p.g_operand_ld + p.K - 1;
          const int s0 = (int)(e0 / p.g_shard_elems), s1 = (int)(e1 / p.g_shard_elems);
          for (int sh = s0; sh <= s1 && ok; ++sh) {
            uint32_t spins = 0;
            while (true) {
              int v;
              asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p.g_ready + sh) : "memory");
              if (v >= p.g_epoch) break;
              if (++spins > GF_WAIT_LIMIT) {
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
        for (int kb = 0; kb < ti.nkb; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1)) {
            set_status(p.status, GF_ERR_WAIT_EMPTY);
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * Cfg::STAGE_BYTES;
          uint8_t* sb = sa + Cfg::A_BYTES;
          mbar_expect_tx(&full_bar[stage], Cfg::STAGE_BYTES);
          const int k0 = ti.k_begin + kb * BK;
          if (!A_MN) {
            int ak = k0, am = m0;
            if (p.conv_cpb > 0) {
              const int kbi = k0 / BK;
              const int tap = kbi / p.conv_cpb;
              const int ky = tap / p.conv_kw, kx = tap - ky * p.conv_kw;
              ak = (kbi - tap * p.conv_cpb) * BK;
              am = m0 + (ky - p.conv_pad) * p.conv_pitch + (kx - p.conv_pad);   // may be negative: zero fill
            }
            tma_load_2d(sa, &tmA, &full_bar[stage], ak, am);
          } else {
#pragma unroll
            for (int c = 0; c < BM / 64; ++c) tma_load_2d(sa + c * (BK * 128), &tmA, &full_bar[stage], m0 + c * 64, k0);
          }
          if (!B_MN) {
            tma_load_2d(sb, &tmB, &full_bar[stage], k0, ti.b_row + n0);
          } else {
#pragma unroll
            for (int c = 0; c < BN / 64; ++c)
              tma_load_2d(sb + c * (BK * 128), &tmB, &full_bar[stage], n0 + c * 64, ti.b_k_add + k0);
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
      for (int tile = cta; tile < num_tiles && ok; tile += nctas) {
        TileInfo ti;
        if (!tile_info(p, tile, num_kb, ti) || ti.nkb == 0) continue;
        const int buf = it & 1;
        const uint32_t bphase = (it >> 1) & 1;
        ++it;
        if (!mbar_wait(&tempty_bar[buf], bphase ^ 1)) {
          set_status(p.status, GF_ERR_WAIT_TMEM_EMPTY);
          break;
        }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + buf * BN;
        for (int kb = 0; kb < ti.nkb; ++kb) {
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
    for (int tile = cta; tile < num_tiles; tile += nctas) {
      TileInfo ti;
      if (!tile_info(p, tile, num_kb, ti)) continue;
      const int tm = ti.tm, tn = ti.tn;
      if (p.grp_mode == 1) ti.c_row_add = 0;
      const int row = tm * BM + lane_grp * 32 + lane;
      const int n0 = tn * BN;
      if (ti.nkb == 0) {
        // empty segment of a grouped weight gradient: the result is zero
        if (!p.accumulate && row < p.M) {
          for (int col = n0; col < min(p.N, n0 + BN); ++col) {
            if (p.out_fp32) reinterpret_cast<float*>(p.C)[(ti.c_row_add + row) * p.ldc + col] = 0.f;
            else reinterpret_cast<__nv_bfloat16*>(p.C)[(ti.c_row_add + row) * p.ldc + col] = __float2bfloat16(0.f);
          }
        }
        continue;
      }
      const int buf = it & 1;
      const uint32_t bphase = (it >> 1) & 1;
      ++it;
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
          if (p.bias && p.rs_world == 0 && p.split_k <= 1) {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (full || col0 + j < p.N) v[j] += __bfloat162float(p.bias[col0 + j]);
          }
          if (p.residual && p.rs_world == 0 && p.split_k <= 1) {
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
          if (p.rs_tma) {
            __nv_bfloat16* stg = reinterpret_cast<__nv_bfloat16*>(rs_stage_smem) + (warp - 2) * 32 * RS_STAGE_COLS;
            const int sub = c & 3;
            if (sub == 0) {
              if (lane == 0) tma_store_wait_read<0>();     // the previous store has read the staging rows
              __syncwarp();
            }
            __nv_bfloat16* sp = stg + lane * RS_STAGE_COLS + sub * 32;
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              uint4 o;
              o.x = pack_bf16x2(v[q * 8 + 0], v[q * 8 + 1]);
              o.y = pack_bf16x2(v[q * 8 + 2], v[q * 8 + 3]);
              o.z = pack_bf16x2(v[q * 8 + 4], v[q * 8 + 5]);
              o.w = pack_bf16x2(v[q * 8 + 6], v[q * 8 + 7]);
              *reinterpret_cast<uint4*>(sp + q * 8) = o;
            }
            if (sub == 3 || col0 + 32 >= p.N) {
              fence_proxy_async_smem();
              __syncwarp();
              if (lane == 0) {
                const int row0 = tm * BM + lane_grp * 32;
                const int owner = row0 / p.rs_rows_per_rank;
                const int srow = p.rs_rank * p.rs_rows_per_rank + (row0 - owner * p.rs_rows_per_rank);
                tma_store_2d(&rsm.m[owner], stg, n0 + (c >> 2) * RS_STAGE_COLS, srow);
                tma_store_commit();
              }
            }
          } else if (p.rs_world > 0) {
            // partial result -> owner's staging slot [my rank][local row]
            const int owner = row / p.rs_rows_per_rank;
            const int lrow = row - owner * p.rs_rows_per_rank;
            __nv_bfloat16* cp = p.rs_stage[owner] + ((long long)p.rs_rank * p.rs_rows_per_rank + lrow) * p.N + col0;
            if (full) {
#pragma unroll
              for (int q = 0; q < 4; ++q) {
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
                if (col0 + j < p.N) cp[j] = __float2bfloat16(v[j]);
            }
          } else if (p.split_k > 1) {
            float* wp = p.ws + (long long)row * p.N + col0;
            if (full && (p.N & 3) == 0) {
#pragma unroll
              for (int q = 0; q < 8; ++q)
                asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(wp + q * 4), "f"(v[q * 4]),
                             "f"(v[q * 4 + 1]), "f"(v[q * 4 + 2]), "f"(v[q * 4 + 3]) : "memory");
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (col0 + j < p.N) atomicAdd(wp + j, v[j]);
            }
          } else if (p.out_fp32) {
            float* cp = reinterpret_cast<float*>(p.C) + (ti.c_row_add + row) * p.ldc + col0;
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
            __nv_bfloat16* cp = reinterpret_cast<__nv_bfloat16*>(p.C) + (ti.c_row_add + row) * p.ldc + col0;
            if (p.sc_ret) {
              const int2 rt = __ldg(p.sc_ret + row);
              if (rt.y < 0) continue;
              if (!GF_CHECK_IDX(p.status, rt.x, p.sc_world, GF_SITE_SCATTER_RANK)) continue;
              cp = p.sc_dst[rt.x] + (long long)rt.y * p.sc_ld + col0;
            }
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
      if (p.rs_world > 0) {
        // all 128 epilogue threads have stored their rows: publish the tile to the owners of those rows
        if (p.rs_tma && lane == 0) tma_store_wait<0>();
        __threadfence_system();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (warp == 2 && lane == 0) {
          const int m0 = tm * BM;
          int m1 = m0 + BM - 1;
          if (m1 > p.M - 1) m1 = p.M - 1;
          for (int o = m0 / p.rs_rows_per_rank; o <= m1 / p.rs_rows_per_rank; ++o)
            asm volatile("red.release.sys.global.add.s32 [%0], %1;" ::"l"(p.rs_counters[o] + tn), "r"(1) : "memory");
        }
      }
    }
  }

  // ------------------------------------------------------------ reduce phase of the fused reduce-scatter
  if (p.rs_world > 0) {
    __shared__ int s_go;
    __syncthreads();
    const int Mr = p.rs_rows_per_rank, o = p.rs_rank;
    const int cnt = ((o + 1) * Mr - 1) / BM - (o * Mr) / BM + 1;   // row tiles that touch my rows
    const int target = (p.rs_call + 1) * p.rs_world * cnt;
    const int row_chunks = (Mr + 31) / 32;
    const __nv_bfloat16* stage = p.rs_stage[o];
    const int* counters = p.rs_counters[o];
    for (int item = cta; item < p.tiles_n * row_chunks; item += nctas) {
      const int tn = item / row_chunks, rc = item % row_chunks;
      if (threadIdx.x == 0) {
        int ok = 0;
        for (uint32_t it = 0; it < GF_WAIT_LIMIT; ++it) {
          int v;
          asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(counters + tn) : "memory");
          if (v >= target) { ok = 1; break; }
          __nanosleep(100);
        }
        if (!ok) set_status(p.status, GF_ERR_WAIT_PEER);
        s_go = ok;
      }
      __syncthreads();
      if (s_go) {
        const int r0 = rc * 32, r1 = min(Mr, r0 + 32);
        const int c0 = tn * BN, c1 = min(p.N, c0 + BN);
        const int vpr = (c1 - c0) >> 3;
        for (int v = threadIdx.x; v < (r1 - r0) * vpr; v += blockDim.x) {
          const int lrow = r0 + v / vpr, col = c0 + (v % vpr) * 8;
          float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
          for (int src = 0; src < p.rs_world; ++src) {
            const uint4 u = *reinterpret_cast<const uint4*>(stage + ((long long)src * Mr + lrow) * p.N + col);
            float2 f0 = unpack_bf16x2(u.x), f1 = unpack_bf16x2(u.y), f2 = unpack_bf16x2(u.z), f3 = unpack_bf16x2(u.w);
            acc[0] += f0.x; acc[1] += f0.y; acc[2] += f1.x; acc[3] += f1.y;
            acc[4] += f2.x; acc[5] += f2.y; acc[6] += f3.x; acc[7] += f3.y;
          }
          if (p.bias) {
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[j] += __bfloat162float(p.bias[col + j]);
          }
          if (p.residual) {
            const uint4 u = *reinterpret_cast<const uint4*>(p.residual + (long long)lrow * p.ldr + col);
            float2 f0 = unpack_bf16x2(u.x), f1 = unpack_bf16x2(u.y), f2 = unpack_bf16x2(u.z), f3 = unpack_bf16x2(u.w);
            acc[0] += f0.x; acc[1] += f0.y; acc[2] += f1.x; acc[3] += f1.y;
            acc[4] += f2.x; acc[5] += f2.y; acc[6] += f3.x; acc[7] += f3.y;
          }
          uint4 ov;
          ov.x = pack_bf16x2(acc[0], acc[1]); ov.y = pack_bf16x2(acc[2], acc[3]);
          ov.z = pack_bf16x2(acc[4], acc[5]); ov.w = pack_bf16x2(acc[6], acc[7]);
          *reinterpret_cast<uint4*>(p.rs_out + (long long)lrow * p.rs_ldo + col) = ov;
        }
      }
      __syncthreads();
    }
  }

  // ------------------------------------------------------------ teardown
  if (p.status && *reinterpret_cast<volatile int*>(p.status) != 0) error_drain_pause();
  if (p.sc_ret) __threadfence_system();      // rows stored into peers' buffers by this thread
  tc_fence_before();
  __syncthreads();
  if (p.sc_ret && threadIdx.x == 0) {
    const int done = atomicAdd(p.sc_counter, 1);
    if (done == nctas - 1) {
      *p.sc_counter = 0;
      __threadfence_system();
      for (int r = 0; r < p.sc_world; ++r)
        asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p.sc_flags[r] + p.sc_rank), "r"(p.sc_epoch) : "memory");
    }
  }
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
}

static RsMaps g_no_rs_maps;   // zero-filled; passed when the launch has no reduce-scatter
static thread_local const RsMaps* g_rs_maps = nullptr;

template <int BN, bool A_MN, bool B_MN>
static int launch_gemm(const CUtensorMap& tmA, const CUtensorMap& tmB, GemmParams& p, int max_ctas,
                       cudaStream_t stream) {
  using Cfg = GemmCfg<BN>;
  static gf::DeviceOnce configured;
  auto kern = gemm_bf16_kernel<BN, A_MN, B_MN>;
  if (configured.todo()) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         Cfg::SMEM_BYTES + RS_STAGE_BYTES);
    if (e != cudaSuccess) return GFH_CUDA;
    configured.mark();
  }
  p.tiles_m = (p.M + BM - 1) / BM;
  p.tiles_n = (p.N + BN - 1) / BN;
  int tiles = p.tiles_m * p.tiles_n * (p.grp_mode == 2 ? p.grp_experts : 1) * (p.split_k > 1 ? p.split_k : 1);
  int grid = sm_count();
  if (max_ctas > 0 && max_ctas < grid) grid = max_ctas;
  const int n_copy = p.g_operand >= 0 ? p.g_copy_ctas : 0;
  if (tiles < grid - n_copy) grid = tiles + n_copy;
  p.group_m = 0;
  // rows of a band of the tile walk; GF_GEMM_BAND overrides the default of 16 (read once, thread-safe)
  static const int band_rows = [] {
    const char* e = getenv("GF_GEMM_BAND");
    const int v = e ? atoi(e) : 16;
    return v < 1 ? 16 : v;
  }();
  const int band = p.tiles_m > band_rows ? band_rows : p.tiles_m;
  if (p.rs_world > 0) {
    // row blocks alternate between owners when every owner has whole row blocks; otherwise start after the own rows
    p.rs_interleave = (p.rs_rows_per_rank % BM == 0) ? p.rs_rows_per_rank / BM : 0;
    const int next = (p.rs_rank + 1) % p.rs_world;
    p.tile_rot = p.rs_interleave ? 0 : (int)(((long long)next * p.rs_rows_per_rank / BM) % p.tiles_m);
    p.group_m = band;
  } else if (p.g_operand == 0) {
    // A is gathered: start the walk in the row blocks of the shard that is copied first (the local one)
    const long long first = p.g_first_shard * p.g_shard_elems - p.g_operand_off;
    const long long row = first > 0 ? (first + p.g_operand_ld - 1) / p.g_operand_ld : 0;
    p.tile_rot = (int)((row / BM) % p.tiles_m);
    p.group_m = band;
  } else if (p.g_operand == 1) {
    // B is gathered: all row blocks of one column block, column blocks starting in the local shard
    const long long first = p.g_first_shard * p.g_shard_elems - p.g_operand_off;
    const long long row = first > 0 ? (first + p.g_operand_ld - 1) / p.g_operand_ld : 0;
    p.order_n_fast = 0;
    p.tile_rot = (int)((row / BN) % p.tiles_n);
  } else if (p.grp_mode != 2 && p.tiles_n > 1) {
    p.group_m = band;
    p.tile_rot = 0;
  }
  const RsMaps* maps = (p.rs_tma && g_rs_maps) ? g_rs_maps : &g_no_rs_maps;
  if (p.rs_tma && !g_rs_maps) p.rs_tma = 0;
  kern<<<grid, GEMM_THREADS, Cfg::SMEM_BYTES + (p.rs_tma ? RS_STAGE_BYTES : 0), stream>>>(tmA, tmB, p, *maps);
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

static int gemm_core(const void* A, const void* B, void* C, int M, int N, int K, int a_mn_major, long long lda,
                     int b_mn_major, long long ldb, long long ldc, int out_fp32, int accumulate, const void* bias,
                     const void* residual, long long ldr, float alpha, int* status, int bn_hint, int max_ctas,
                     gf::GemmParams& p, cudaStream_t stream) {
  using namespace gf;
  if (M <= 0 || N <= 0 || K <= 0) return GFH_BAD_ARG;
  const int bn = pick_bn(M, N, bn_hint);
  CUtensorMap tmA, tmB;
  int rc;
  if (!a_mn_major)   // implicit convolution: the map covers the [rows, C] image, not an unfolded [rows, taps * C]
    rc = make_tmap_2d(&tmA, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, M, p.conv_cpb > 0 ? p.conv_cpb * BK : K, lda * 2,
                      BM, BK);
  else
    rc = make_tmap_2d(&tmA, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, M, lda * 2, BK, 64);
  if (rc) return rc;
  const long long stack = p.grp_mode == 1 ? p.grp_experts : 1;   // B is `stack` matrices one after another
  if (!b_mn_major)
    rc = make_tmap_2d(&tmB, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, N * stack, K, ldb * 2, bn, BK);
  else
    rc = make_tmap_2d(&tmB, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K * stack, N, ldb * 2, BK, 64);
  if (rc) return rc;
  p.M = M; p.N = N; p.K = K;
  p.C = C; p.ldc = ldc; p.out_fp32 = out_fp32; p.accumulate = accumulate;
  p.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  p.residual = reinterpret_cast<const __nv_bfloat16*>(residual);
  p.ldr = ldr; p.alpha = alpha; p.status = status;
#define GF_DISPATCH(BN_)                                                                  \
  if (!a_mn_major && !b_mn_major) return launch_gemm<BN_, false, false>(tmA, tmB, p, max_ctas, stream); \
  if (!a_mn_major && b_mn_major) return launch_gemm<BN_, false, true>(tmA, tmB, p, max_ctas, stream);   \
  if (a_mn_major && !b_mn_major) return launch_gemm<BN_, true, false>(tmA, tmB, p, max_ctas, stream);   \
  return launch_gemm<BN_, true, true>(tmA, tmB, p, max_ctas, stream);
  if (bn == 256) { GF_DISPATCH(256) }
  GF_DISPATCH(128)
#undef GF_DISPATCH
}

namespace gf {
// C = bf16(ws + bias + residual); ws is the fp32 sum of the k slices (alpha already applied).
__global__ void splitk_finish_kernel(const float* __restrict__ ws, __nv_bfloat16* __restrict__ C, long long ldc,
                                     const __nv_bfloat16* __restrict__ bias, const __nv_bfloat16* __restrict__ residual,
                                     long long ldr, int M, int N) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long long)M * N) return;
  const int r = (int)(i / N), c = (int)(i % N);
  float v = ws[i];
  if (bias) v += __bfloat162float(bias[c]);
  if (residual) v += __bfloat162float(residual[(long long)r * ldr + c]);
  C[(long long)r * ldc + c] = __float2bfloat16(v);
}

// fp32 workspace per device, grown on demand and kept. Calls that use it on different streams of one device must
// not overlap (the training engines issue GEMMs on one stream per device).
static float* g_splitk_ws[32] = {};
static size_t g_splitk_cap[32] = {};
static float* splitk_workspace(size_t floats) {
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 32) return nullptr;
  if (g_splitk_cap[dev] < floats) {
    if (g_splitk_ws[dev]) cudaFree(g_splitk_ws[dev]);
    size_t cap = floats < (size_t)(8 << 20) ? (size_t)(8 << 20) : floats;
    if (cudaMalloc(&g_splitk_ws[dev], cap * sizeof(float)) != cudaSuccess) {
      g_splitk_ws[dev] = nullptr;
      g_splitk_cap[dev] = 0;
      cudaGetLastError();
      return nullptr;
    }
    g_splitk_cap[dev] = cap;
  }
  return g_splitk_ws[dev];
}
}  // namespace gf

namespace gf {
// CTA-pair kernel for plain GEMMs (gemm2sm_bf16.cu)
int gemm2sm_wanted(int M, int N, int K);
int gemm2sm_run(const void* A, const void* B, void* C, int M, int N, int K, int a_mn_major, long long lda,
                int b_mn_major, long long ldb, long long ldc, int out_fp32, int accumulate, const void* bias,
                const void* residual, long long ldr, float alpha, int* status, int activation, cudaStream_t stream);
}  // namespace gf

static void no_gather(gf::GemmParams& p) {
  p.g_operand = -1; p.g_copy_ctas = 0; p.g_world = 1; p.g_rank = 0; p.g_first_shard = 0;
  for (int i = 0; i < 8; ++i) p.g_src[i] = nullptr;
  p.g_dst = nullptr; p.g_shard_elems = 8; p.g_operand_off = 0; p.g_operand_ld = 1; p.g_ready = nullptr;
  p.g_counters = nullptr; p.g_epoch = 0; p.g_version_pad = nullptr; p.g_version_idx = 0; p.g_version_val = 0;
  p.order_n_fast = 0; p.tile_rot = 0; p.rs_interleave = 0; p.rs_tma = 0;
  p.grp_offsets = nullptr; p.grp_experts = 0; p.grp_mode = 0; p.grp_b_rows = 0; p.split_k = 1; p.ws = nullptr; p.act = 0;
  p.grp_src_start = nullptr; p.grp_arrived = nullptr; p.grp_world = 1; p.grp_epoch = 0;
  p.sc_ret = nullptr; p.sc_ld = 0; p.sc_world = 0; p.sc_rank = 0; p.sc_epoch = 0; p.sc_counter = nullptr;
  for (int i = 0; i < 8; ++i) { p.sc_dst[i] = nullptr; p.sc_flags[i] = nullptr; }
  p.rs_world = 0; p.rs_rank = 0; p.rs_rows_per_rank = 1; p.rs_call = 0; p.rs_out = nullptr; p.rs_ldo = 0;
  for (int i = 0; i < 8; ++i) { p.rs_stage[i] = nullptr; p.rs_counters[i] = nullptr; }
  p.conv_cpb = 0; p.conv_kw = 1; p.conv_pitch = 0; p.conv_pad = 0;
}

// lda/ldb: row pitch in elements of the matrix as stored.
//   a_mn_major = 0: A stored [M, K] (K contiguous); 1: A stored [K, M] (M contiguous).
//   b_mn_major = 0: B stored [N, K] (K contiguous); 1: B stored [K, N] (N contiguous).
GF_API int gf_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, int a_mn_major, long long lda,
                        int b_mn_major, long long ldb, long long ldc, int out_fp32, int accumulate,
                        const void* bias, const void* residual, long long ldr, float alpha, int* status,
                        int bn_hint, int max_ctas, const int* splitk_ws, int activation, int splitk_ws_floats,
                        void* stream_v) {
  gf::enter();
  gf::GemmParams p;
  no_gather(p);
  p.act = activation == 1 ? 1 : 0;   // epilogue activation after bias and residual: 0 none, 1 ReLU
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream_v);
  // Few output tiles and a long K (decode-sized M; weight gradients of narrow layers, [768, 2304] over 8192 tokens):
  // too few tiles to fill the machine. Split K until there is about one work item per SM; the slices add into an
  // fp32 workspace that a second kernel converts. The workspace is the caller's (splitk_ws, splitk_ws_floats >= M * N:
  // a buffer that belongs to the calling stream, e.g. from a stream-ordered allocator) or, without one, a buffer
  // this library keeps per device, which only one stream at a time may use.
  const int bn_sk = N <= 128 ? 128 : 256;
  const long long tiles_sk = (long long)((M + gf::BM - 1) / gf::BM) * ((N + bn_sk - 1) / bn_sk);
  if (tiles_sk * 2 <= gf::sm_count() && !out_fp32 && !accumulate && K >= 2048 && bn_hint == 0 && max_ctas == 0 &&
      p.act == 0) {
    const int bn = bn_sk;
    const long long tiles = tiles_sk;
    const int sms = gf::sm_count();
    int split = (int)(sms / (tiles > 0 ? tiles : 1));
    if (split > K / 512) split = K / 512;
    if (split > 16) split = 16;
    if (split >= 2) {
      float* ws = (splitk_ws && (long long)splitk_ws_floats >= (long long)M * N)
                      ? reinterpret_cast<float*>(const_cast<int*>(splitk_ws))
                      : gf::splitk_workspace((size_t)M * N);
      if (ws) {
        if (cudaMemsetAsync(ws, 0, sizeof(float) * (size_t)M * N, st) != cudaSuccess) return gf::GFH_CUDA;
        p.split_k = split;
        p.ws = ws;
        int rc = gemm_core(A, B, C, M, N, K, a_mn_major, lda, b_mn_major, ldb, ldc, 0, 0, nullptr, nullptr, 0, alpha,
                           status, bn, 0, p, st);
        if (rc) return rc;
        const long long n = (long long)M * N;
        gf::splitk_finish_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(
            ws, reinterpret_cast<__nv_bfloat16*>(C), ldc, reinterpret_cast<const __nv_bfloat16*>(bias),
            reinterpret_cast<const __nv_bfloat16*>(residual), ldr, M, N);
        gf::note_extra_launches(1);
        return cudaGetLastError() == cudaSuccess ? gf::GFH_OK : gf::GFH_CUDA;
      }
    }
  }
  // large plain products run on CTA pairs (256 x 256 tiles, half the operand bytes per SM and flop)
  if (bn_hint == 0 && max_ctas == 0 && gf::gemm2sm_wanted(M, N, K))
    return gf::gemm2sm_run(A, B, C, M, N, K, a_mn_major, lda, b_mn_major, ldb, ldc, out_fp32, accumulate, bias,
                           residual, ldr, alpha, status, activation, st);
  return gemm_core(A, B, C, M, N, K, a_mn_major, lda, b_mn_major, ldb, ldc, out_fp32, accumulate, bias, residual, ldr,
                   alpha, status, bn_hint, max_ctas, p, st);
}

// Stride-1 "same" convolution without unfolding: Y[rows, Cout] = act(conv(Xp) + bias) on the padded pixel grid.
//   Xp  bf16 [rows, C], rows = images * (H + pad) * (W + pad): channels-last pixels, `pad` zero pixels after every
//       image row and `pad` zero rows after every image (pad = (window - 1) / 2), C a multiple of 64
//   Wt  bf16 [Cout, KH * KW * C], tap-major, channel-minor
//   Y   bf16 [rows, Cout]: rows of padding pixels hold values that mean nothing; the caller drops them
//   residual (optional) bf16 [rows, Cout] on the same padded grid, added before the activation
// One GEMM with K = KH * KW * C whose A tiles are row-shifted reads of Xp (see GemmParams::conv_*).
GF_API int gf_conv_implicit_bf16(const void* Xp, const void* Wt, void* Y, long long rows, int C, int Cout, int KH,
                                 int KW, int pitch, const void* bias, const void* residual, int relu, int* status,
                                 void* stream_v) {
  gf::enter();
  if (rows <= 0 || rows > 0x7fffffffLL || C <= 0 || C % gf::BK || Cout <= 0 || Cout % 8 || KH != KW || !(KH & 1) ||
      pitch <= (KW - 1) / 2)
    return gf::GFH_BAD_ARG;
  gf::GemmParams p;
  no_gather(p);
  p.act = relu ? 1 : 0;
  p.conv_cpb = C / gf::BK; p.conv_kw = KW; p.conv_pitch = pitch; p.conv_pad = (KW - 1) / 2;
  const int K = KH * KW * C;
  return gemm_core(Xp, Wt, Y, (int)rows, Cout, K, 0, C, 0, K, Cout, 0, 0, bias, residual, Cout, 1.f, status, 0, 0, p,
                   reinterpret_cast<cudaStream_t>(stream_v));
}

// Grouped GEMM over the row segments of a row-sorted buffer (the experts of a mixture-of-experts layer).
// `offsets` is a DEVICE int[experts + 1]: first row of every segment and the total; every entry must be a multiple
// of 128 and rows between a segment's last token and the next boundary must hold zeros.
//   mode 1: C[rows, N] = A[rows, K] * op(B_e) for the rows of segment e. A is K-major with `rows_cap` rows
//           (an upper bound of offsets[experts]; tiles beyond the total are skipped). B is the stacked weight:
//           b_mn_major = 0 -> [experts, N, K]; 1 -> [experts, K, N].
//   mode 2: C_e[M, N] = A[rows_e, M]^T * B[rows_e, N] (both operands row-sorted activations, MN-major), C stacked
//           [experts, M, N]; `rows_cap` is the row count of A and B.
GF_API int gf_gemm_bf16_grouped(const void* A, const void* B, void* C, int mode, int rows_cap, int M, int N, int K,
                                long long lda, int b_mn_major, long long ldb, long long ldc, int out_fp32,
                                int accumulate, float alpha, int* status, const int* offsets, int experts,
                                const int* src_start, const int* arrived, int world, int epoch,
                                const void* scatter_ret, const unsigned long long* scatter_dst,
                                const unsigned long long* scatter_flags, long long scatter_ld, int my_rank,
                                int scatter_epoch, int* scatter_counter, void* stream_v) {
  gf::enter();
  if (!offsets || experts <= 0 || (mode != 1 && mode != 2) || rows_cap % 128) return gf::GFH_BAD_ARG;
  if (world < 1 || world > 8) return gf::GFH_BAD_ARG;
  gf::GemmParams p;
  no_gather(p);
  p.grp_offsets = offsets; p.grp_experts = experts; p.grp_mode = mode;
  if (src_start && arrived) {
    p.grp_src_start = src_start; p.grp_arrived = arrived; p.grp_world = world; p.grp_epoch = epoch;
  }
  if (scatter_ret) {
    if (mode != 1 || out_fp32 || accumulate || !scatter_dst || !scatter_flags || !scatter_counter)
      return gf::GFH_BAD_ARG;
    p.sc_ret = reinterpret_cast<const int2*>(scatter_ret);
    for (int i = 0; i < world; ++i) {
      p.sc_dst[i] = reinterpret_cast<__nv_bfloat16*>(scatter_dst[i]);
      p.sc_flags[i] = reinterpret_cast<int*>(scatter_flags[i]);
    }
    p.sc_ld = scatter_ld; p.sc_world = world; p.sc_rank = my_rank; p.sc_epoch = scatter_epoch;
    p.sc_counter = scatter_counter;
  }
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream_v);
  if (mode == 1) {
    p.grp_b_rows = b_mn_major ? K : N;
    return gemm_core(A, B, C, rows_cap, N, K, 0, lda, b_mn_major, ldb, ldc, out_fp32, accumulate, nullptr, nullptr, 0,
                     alpha, status, 0, 0, p, st);
  }
  return gemm_core(A, B, C, M, N, rows_cap, 1, lda, 1, ldb, ldc, out_fp32, accumulate, nullptr, nullptr, 0, alpha,
                   status, 0, 0, p, st);
}

// Fused all-gather + GEMM. `operand` = 0: A ([M, K], K-major) is a view into the gathered buffer `g_dst`;
// 1: B ([N, K], K-major) is. `src_ptrs` are every rank's shard of that buffer (world pointers, peer-mapped);
// the kernel's first `copy_ctas` CTAs copy them into g_dst while the others compute. `ready` and `counters`
// are local int[world] (counters zero); `epoch` must grow with every call that reuses `ready`. Shards are copied
// in the order first_shard, first_shard + 1, ... (first_shard < 0: this rank's own shard first).
GF_API int gf_gemm_bf16_allgather(const void* A, const void* B, void* C, int M, int N, int K, long long lda,
                                  long long ldb, long long ldc, int out_fp32, const void* bias, const void* residual,
                                  long long ldr, float alpha, int* status, int operand,
                                  const unsigned long long* src_ptrs, void* g_dst, long long shard_elems, int world,
                                  int my_rank, int first_shard, int copy_ctas, int* ready, int* counters, int epoch,
                                  const int* version_pad, int version_idx, int version_val, void* stream_v) {
  gf::enter();
  if (world < 1 || world > 8 || (shard_elems & 7) || copy_ctas < 1 || (operand != 0 && operand != 1)) return gf::GFH_BAD_ARG;
  gf::GemmParams p;
  no_gather(p);
  p.g_operand = operand; p.g_copy_ctas = copy_ctas; p.g_world = world; p.g_rank = my_rank;
  p.g_first_shard = (first_shard >= 0 && first_shard < world) ? first_shard : my_rank;
  for (int i = 0; i < world; ++i) p.g_src[i] = reinterpret_cast<const void*>(src_ptrs[i]);
  p.g_dst = reinterpret_cast<__nv_bfloat16*>(g_dst);
  p.g_shard_elems = shard_elems;
  const char* opnd = reinterpret_cast<const char*>(operand == 0 ? A : B);
  p.g_operand_off = (opnd - reinterpret_cast<const char*>(g_dst)) / 2;
  p.g_operand_ld = operand == 0 ? lda : ldb;
  if (p.g_operand_off < 0) return gf::GFH_BAD_ARG;
  p.g_ready = ready; p.g_counters = counters; p.g_epoch = epoch;
  p.g_version_pad = version_pad; p.g_version_idx = version_idx; p.g_version_val = version_val;
  return gemm_core(A, B, C, M, N, K, 0, lda, 0, ldb, ldc, out_fp32, 0, bias, residual, ldr, alpha, status, 256, 0, p,
                   reinterpret_cast<cudaStream_t>(stream_v));
}

// Fused GEMM + reduce-scatter for a row-parallel linear: every rank passes its partial operands
// (A [M, K_local] K-major, B [N, K_local] K-major). Rows of the result are owned in blocks of M / world; this
// rank's block (sum over ranks, + bias, + residual [M / world, N]) lands in `out`. `stage_ptrs` / `counter_ptrs`
// are every rank's staging buffer ([world, M / world, N] bf16) and arrival counters (int[ceil(N / 256)], zeroed
// once); `call_index` counts earlier calls on the same counters with the same shape.
GF_API int gf_gemm_bf16_reduce_scatter(const void* A, const void* B, void* out, int M, int N, int K, long long lda,
                                       long long ldb, long long ldo, const void* bias, const void* residual,
                                       long long ldr, float alpha, int* status, const unsigned long long* stage_ptrs,
                                       const unsigned long long* counter_ptrs, int world, int my_rank, int call_index,
                                       int max_ctas, void* stream_v) {
  gf::enter();
  if (world < 1 || world > 8 || (M % world) || (N & 7) || (ldo & 7)) return gf::GFH_BAD_ARG;
  gf::GemmParams p;
  no_gather(p);
  p.rs_world = world; p.rs_rank = my_rank; p.rs_rows_per_rank = M / world; p.rs_call = call_index;
  p.rs_out = reinterpret_cast<__nv_bfloat16*>(out); p.rs_ldo = ldo;
  for (int i = 0; i < world; ++i) {
    p.rs_stage[i] = reinterpret_cast<__nv_bfloat16*>(stage_ptrs[i]);
    p.rs_counters[i] = reinterpret_cast<int*>(counter_ptrs[i]);
  }
  gf::RsMaps maps;
  if ((M / world) % gf::BM == 0) {
    // partial tiles go out as TMA stores of 32 x 128 boxes into the owners' staging buffers
    p.rs_tma = 1;
    for (int i = 0; i < 8; ++i) {
      const int src = i < world ? i : 0;
      int rc = gf::make_tmap_2d(&maps.m[i], reinterpret_cast<const void*>(stage_ptrs[src]),
                                CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, M, N, (long long)N * 2, 32, gf::RS_STAGE_COLS,
                                CU_TENSOR_MAP_SWIZZLE_NONE);
      if (rc) return rc;
    }
    gf::g_rs_maps = &maps;
  }
  int rc = gemm_core(A, B, out, M, N, K, 0, lda, 0, ldb, ldo, 0, 0, bias, residual, ldr, alpha, status, 256, max_ctas,
                     p, reinterpret_cast<cudaStream_t>(stream_v));
  gf::g_rs_maps = nullptr;
  return rc;
}
