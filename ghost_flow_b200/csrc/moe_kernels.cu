// Mixture-of-experts routing and the all-to-all dispatch / combine over peer memory.
//
// The reference routes token by token on the CPU (ghostflow-nn/src/mixture_of_experts.rs:152-177 router with
// softmax + top-k, :212-274 per-token expert loop, :289-323 load-balance loss) and has no expert parallelism.
// Here the experts are sharded over the ranks of one NVSwitch box and every step is a kernel:
//
//   route      softmax + top-k (+ renormalisation) per token, one warp per token, expert histogram
//   publish    this rank's histogram -> every rank's count table (peer stores + release flag)
//   plan       one CTA: waits (bounded) for all histograms, lays out every expert's row segment (rows sorted by
//              source rank, segment starts padded to 128 rows for the grouped GEMM)
//   dispatch   one warp per (token, slot): copies the token row straight into the owner rank's segment over
//              NVLink, records where the result has to come back to, signals arrival per source rank
//   zero_pad   zeroes the padding rows of the local segments
//   combine    waits (bounded) for every rank's expert outputs and forms the weighted sum per token
//
// The expert GEMMs in between are gf_gemm_bf16_grouped: its producer waits per tile for the source ranks whose
// rows the tile reads, and its epilogue can store output rows directly into the token's home rank (the combine
// all-to-all fused into the GEMM).
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "gf_host.h"
#include "gf_ptx.cuh"

namespace gf {

struct Peers {
  void* p[8];
};

constexpr int MOE_MAX_E = 256;

// ------------------------------------------------------------------ route
// logits [T, E] (bf16 or fp32). idx [T, k], w [T, k] fp32, probs [T, E] fp32 (optional), counts [E] (+= per token).
__global__ void moe_route_kernel(const void* __restrict__ logits, int logits_f32, int T, int E, int k, int renorm,
                                 int* __restrict__ idx, float* __restrict__ w, float* __restrict__ probs,
                                 int* __restrict__ counts) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= T) return;
  float v[MOE_MAX_E / 32];
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < MOE_MAX_E / 32; ++i) {
    const int e = lane + i * 32;
    float x = -INFINITY;
    if (e < E)
      x = logits_f32 ? reinterpret_cast<const float*>(logits)[(long long)warp * E + e]
                     : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(logits)[(long long)warp * E + e]);
    v[i] = x;
    mx = fmaxf(mx, x);
  }
  for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < MOE_MAX_E / 32; ++i) {
    v[i] = (lane + i * 32 < E) ? __expf(v[i] - mx) : 0.f;
    sum += v[i];
  }
  for (int o = 16; o; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  const float inv = 1.f / sum;
#pragma unroll
  for (int i = 0; i < MOE_MAX_E / 32; ++i) {
    v[i] *= inv;
    if (probs && lane + i * 32 < E) probs[(long long)warp * E + lane + i * 32] = v[i];
  }
  float sel_sum = 0.f;
  float my_w = 0.f;
  int my_e = 0;
  for (int s = 0; s < k; ++s) {
    float best = -1.f;
    int be = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < MOE_MAX_E / 32; ++i)
      if (v[i] > best) { best = v[i]; be = lane + i * 32; }
    for (int o = 16; o; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oe = __shfl_xor_sync(0xffffffffu, be, o);
      if (ob > best || (ob == best && oe < be)) { best = ob; be = oe; }
    }
    if ((be & 31) == lane) v[be >> 5] = -2.f;   // taken
    sel_sum += best;
    if (lane == s) { my_w = best; my_e = be; }
  }
  if (lane < k) {
    idx[(long long)warp * k + lane] = my_e;
    w[(long long)warp * k + lane] = renorm ? my_w / sel_sum : my_w;
    atomicAdd(counts + my_e, 1);
  }
}

// ------------------------------------------------------------------ publish
__global__ void moe_publish_kernel(Peers tables, Peers flags, const int* __restrict__ counts, int E, int world,
                                   int rank, int flag_row, int epoch) {
  // CTA r writes this rank's histogram into rank r's table row [rank], then releases the flag
  const int r = blockIdx.x;
  int* dst = reinterpret_cast<int*>(tables.p[r]) + rank * E;
  for (int e = threadIdx.x; e < E; e += blockDim.x) dst[e] = counts[e];
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0)
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(reinterpret_cast<int*>(flags.p[r]) + flag_row * 8 + rank),
                 "r"(epoch) : "memory");
}

// ------------------------------------------------------------------ plan
// table [world, E] (local). Outputs (all local):
//   seg_offsets [E_local + 1]  padded segment starts of this rank's experts
//   src_start   [E_local, world + 1]  first row of each source rank inside each local segment (last = end of tokens)
//   send_base   [E]  row in the OWNER's buffer where this rank's tokens of expert e start
//   cursor      [E]  zeroed
__global__ void moe_plan_kernel(const int* __restrict__ table, const int* __restrict__ flags, int flag_row, int epoch,
                                int E, int world, int rank, int rows_cap, int* __restrict__ seg_offsets,
                                int* __restrict__ src_start, int* __restrict__ send_base, int* __restrict__ cursor,
                                int* status) {
  __shared__ int ok;
  if (threadIdx.x == 0) {
    ok = 1;
    for (int r = 0; r < world && ok; ++r) {
      uint32_t spins = 0;
      while (true) {
        int v;
        asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(flags + flag_row * 8 + r) : "memory");
        if (v >= epoch) break;
        if (++spins > GF_WAIT_LIMIT) { ok = 0; break; }
        __nanosleep(64);
      }
    }
    if (!ok && status) atomicCAS(status, 0, GF_ERR_WAIT_PEER);
  }
  __syncthreads();
  if (threadIdx.x != 0) return;
  const int el = E / world;
  for (int owner = 0; owner < world; ++owner) {
    int off = 0;
    for (int j = 0; j < el; ++j) {
      const int e = owner * el + j;
      int run = off;
      for (int r = 0; r < world; ++r) {
        const int c = ok ? table[r * E + e] : 0;
        if (owner == rank) src_start[j * (world + 1) + r] = run;
        if (r == rank) send_base[e] = run;
        run += c;
      }
      if (owner == rank) {
        src_start[j * (world + 1) + world] = run;
        seg_offsets[j] = off;
      }
      off = (run + 127) & ~127;
      cursor[e] = 0;
    }
    if (owner == rank) {
      seg_offsets[el] = off;
      if (off > rows_cap && status) atomicCAS(status, 0, GF_ERR_CAPACITY);
    }
  }
}

// ------------------------------------------------------------------ dispatch
// One warp per (token, slot). mode 0: take the next position of the expert (forward); mode 1: reuse dest_row
// (backward: gradient rows must line up with the forward rows). `scale` (optional, [T*k]) multiplies the row.
__global__ void moe_dispatch_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, const int* __restrict__ idx,
                                    const float* __restrict__ scale, int T, int k, int K, int E, int world, int rank,
                                    int rows_cap, const int* __restrict__ send_base, int* __restrict__ cursor,
                                    int* __restrict__ dest_row, int reuse_rows, Peers bufs, Peers rets, Peers flags,
                                    int flag_row, int epoch, int* done_counter, int* chk) {
  const int lane = threadIdx.x & 31;
  const int wpb = blockDim.x >> 5;
  const int el = E / world;
  (void)chk;
  for (int pair = blockIdx.x * wpb + (threadIdx.x >> 5); pair < T * k; pair += gridDim.x * wpb) {
    const int t = pair / k;
    const int e = idx[pair];
    if (!GF_CHECK_IDX(chk, e, E, GF_SITE_DISPATCH_EXPERT)) continue;
    int row;
    if (reuse_rows) {
      row = dest_row[pair];
    } else {
      int pos = 0;
      if (lane == 0) pos = atomicAdd(cursor + e, 1);
      pos = __shfl_sync(0xffffffffu, pos, 0);
      row = send_base[e] + pos;
      if (lane == 0) dest_row[pair] = row;
    }
    if (row >= rows_cap) continue;            // capacity overflow is reported by the owner's plan kernel
    if (!GF_CHECK_IDX(chk, row, rows_cap, GF_SITE_DISPATCH_ROW)) continue;   // a negative row: corrupted table
    const int owner = e / el;
    __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(bufs.p[owner]) + (long long)row * K;
    const __nv_bfloat16* src = x + (long long)t * ldx;
    const float sc = scale ? scale[pair] : 1.f;
    for (int c = lane * 8; c < K; c += 256) {
      uint4 u = *reinterpret_cast<const uint4*>(src + c);
      if (scale) {
        float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), cc = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
        u.x = pack_bf16x2(a.x * sc, a.y * sc); u.y = pack_bf16x2(b.x * sc, b.y * sc);
        u.z = pack_bf16x2(cc.x * sc, cc.y * sc); u.w = pack_bf16x2(d.x * sc, d.y * sc);
      }
      *reinterpret_cast<uint4*>(dst + c) = u;
    }
    if (lane == 0 && !reuse_rows) reinterpret_cast<int2*>(rets.p[owner])[row] = make_int2(rank, pair);
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int done = atomicAdd(done_counter, 1);
    if (done == (int)gridDim.x - 1) {
      *done_counter = 0;
      __threadfence_system();
      for (int r = 0; r < world; ++r)
        asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(reinterpret_cast<int*>(flags.p[r]) + flag_row * 8 + rank),
                     "r"(epoch) : "memory");
    }
  }
}

// ------------------------------------------------------------------ zero the padding rows
__global__ void moe_zero_pad_kernel(__nv_bfloat16* __restrict__ buf, int K, int2* __restrict__ ret,
                                    const int* __restrict__ seg_offsets, const int* __restrict__ src_start, int el,
                                    int world, int rows_cap) {
  const int j = blockIdx.y;
  const int r0 = src_start[j * (world + 1) + world];
  int r1 = seg_offsets[j + 1];
  if (r1 > rows_cap) r1 = rows_cap;
  for (int row = r0 + blockIdx.x; row < r1; row += gridDim.x) {
    for (int c = threadIdx.x * 8; c < K; c += blockDim.x * 8)
      *reinterpret_cast<uint4*>(buf + (long long)row * K + c) = make_uint4(0, 0, 0, 0);
    if (ret && threadIdx.x == 0) ret[row] = make_int2(0, -1);
  }
}

// ------------------------------------------------------------------ combine
// y[t] = sum_slot w[t, slot] * comb[t * k + slot] (+ residual[t]); w == nullptr: plain sum. Waits for the flags of
// all ranks first. dots (optional, [T * k]) = <g[t], comb[t * k + slot]> for the router gradient.
__global__ void moe_combine_kernel(const __nv_bfloat16* __restrict__ comb, const float* __restrict__ w,
                                   const __nv_bfloat16* __restrict__ residual, __nv_bfloat16* __restrict__ y, int T,
                                   int k, int K, const int* __restrict__ flags, int flag_row, int epoch, int world,
                                   const __nv_bfloat16* __restrict__ g, float* __restrict__ dots, int* status) {
  __shared__ int ok;
  if (flags) {
    if (threadIdx.x == 0) {
      ok = 1;
      for (int r = 0; r < world && ok; ++r) {
        uint32_t spins = 0;
        while (true) {
          int v;
          asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(flags + flag_row * 8 + r) : "memory");
          if (v >= epoch) break;
          if (++spins > GF_WAIT_LIMIT) { ok = 0; break; }
          __nanosleep(64);
        }
      }
      if (!ok && status) atomicCAS(status, 0, GF_ERR_WAIT_PEER);
    }
    __syncthreads();
    if (!ok) return;
  }
  const int lane = threadIdx.x & 31;
  const int wpb = blockDim.x >> 5;
  for (int t = blockIdx.x * wpb + (threadIdx.x >> 5); t < T; t += gridDim.x * wpb) {
    float dot[8];
#pragma unroll
    for (int s = 0; s < 8; ++s) dot[s] = 0.f;
    for (int c = lane * 8; c < K; c += 256) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      float gv[8];
      if (dots) {
        const uint4 u = *reinterpret_cast<const uint4*>(g + (long long)t * K + c);
        float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), cc = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
        gv[0] = a.x; gv[1] = a.y; gv[2] = b.x; gv[3] = b.y; gv[4] = cc.x; gv[5] = cc.y; gv[6] = d.x; gv[7] = d.y;
      }
      for (int s = 0; s < k; ++s) {
        const uint4 u = *reinterpret_cast<const uint4*>(comb + ((long long)t * k + s) * K + c);
        const float ws = w ? w[(long long)t * k + s] : 1.f;
        float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), cc = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
        const float f[8] = {a.x, a.y, b.x, b.y, cc.x, cc.y, d.x, d.y};
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          acc[j] += ws * f[j];
          if (dots && s < 8) dot[s] += gv[j] * f[j];
        }
      }
      if (y) {
        if (residual) {
          const uint4 u = *reinterpret_cast<const uint4*>(residual + (long long)t * K + c);
          float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), cc = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
          acc[0] += a.x; acc[1] += a.y; acc[2] += b.x; acc[3] += b.y;
          acc[4] += cc.x; acc[5] += cc.y; acc[6] += d.x; acc[7] += d.y;
        }
        uint4 o;
        o.x = pack_bf16x2(acc[0], acc[1]); o.y = pack_bf16x2(acc[2], acc[3]);
        o.z = pack_bf16x2(acc[4], acc[5]); o.w = pack_bf16x2(acc[6], acc[7]);
        *reinterpret_cast<uint4*>(y + (long long)t * K + c) = o;
      }
    }
    if (dots) {
      for (int s = 0; s < k && s < 8; ++s) {
        float d = dot[s];
        for (int o = 16; o; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
        if (lane == 0) dots[(long long)t * k + s] = d;
      }
    }
  }
}

static Peers to_peers(const unsigned long long* v, int n) {
  Peers p;
  for (int i = 0; i < 8; ++i) p.p[i] = i < n ? reinterpret_cast<void*>(v[i]) : nullptr;
  return p;
}

}  // namespace gf

using namespace gf;

GF_API int gf_moe_route(const void* logits, int logits_f32, int T, int E, int k, int renorm, int* idx, float* w,
                        float* probs, int* counts, void* stream) {
  gf::enter();
  if (T <= 0 || E <= 0 || E > MOE_MAX_E || k <= 0 || k > 8 || k > E) return GFH_BAD_ARG;
  const int wpb = 8;
  moe_route_kernel<<<(T + wpb - 1) / wpb, wpb * 32, 0, (cudaStream_t)stream>>>(logits, logits_f32, T, E, k, renorm, idx,
                                                                             w, probs, counts);
  return cudaGetLastError() == cudaSuccess ? GFH_OK : GFH_CUDA;
}

GF_API int gf_moe_publish(const unsigned long long* tables, const unsigned long long* flags, const int* counts, int E,
                          int world, int rank, int flag_row, int epoch, void* stream) {
  gf::enter();
  if (world < 1 || world > 8) return GFH_BAD_ARG;
  moe_publish_kernel<<<world, 128, 0, (cudaStream_t)stream>>>(to_peers(tables, world), to_peers(flags, world), counts, E,
                                                              world, rank, flag_row, epoch);
  return cudaGetLastError() == cudaSuccess ? GFH_OK : GFH_CUDA;
}

GF_API int gf_moe_plan(const int* table, const int* flags, int flag_row, int epoch, int E, int world, int rank,
                       int rows_cap, int* seg_offsets, int* src_start, int* send_base, int* cursor, int* status,
                       void* stream) {
  gf::enter();
  if (world < 1 || world > 8 || E % world) return GFH_BAD_ARG;
  moe_plan_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(table, flags, flag_row, epoch, E, world, rank, rows_cap,
                                                      seg_offsets, src_start, send_base, cursor, status);
  return cudaGetLastError() == cudaSuccess ? GFH_OK : GFH_CUDA;
}

GF_API int gf_moe_dispatch(const void* x, long long ldx, const int* idx, const float* scale, int T, int k, int K, int E,
                           int world, int rank, int rows_cap, const int* send_base, int* cursor, int* dest_row,
                           int reuse_rows, const unsigned long long* bufs, const unsigned long long* rets,
                           const unsigned long long* flags, int flag_row, int epoch, int* done_counter,
                           void* stream) {
  gf::enter();
  if (world < 1 || world > 8 || K % 8 || ldx % 8) return GFH_BAD_ARG;
  const int wpb = 8;
  int grid = (T * k + wpb - 1) / wpb;
  const int cap = gf::sm_count() * 4;
  if (grid > cap) grid = cap;
  moe_dispatch_kernel<<<grid, wpb * 32, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)x, ldx, idx, scale, T, k, K, E, world, rank, rows_cap, send_base, cursor, dest_row,
      reuse_rows, to_peers(bufs, world), to_peers(rets, world), to_peers(flags, world), flag_row, epoch, done_counter,
      gf::check_buffer());
  return cudaGetLastError() == cudaSuccess ? GFH_OK : GFH_CUDA;
}

GF_API int gf_moe_zero_pad(void* buf, int K, void* ret, const int* seg_offsets, const int* src_start, int experts_local,
                           int world, int rows_cap, void* stream) {
  gf::enter();
  if (K % 8) return GFH_BAD_ARG;
  moe_zero_pad_kernel<<<dim3(32, experts_local), 128, 0, (cudaStream_t)stream>>>(
      (__nv_bfloat16*)buf, K, (int2*)ret, seg_offsets, src_start, experts_local, world, rows_cap);
  return cudaGetLastError() == cudaSuccess ? GFH_OK : GFH_CUDA;
}

GF_API int gf_moe_combine(const void* comb, const float* w, const void* residual, void* y, int T, int k, int K,
                          const int* flags, int flag_row, int epoch, int world, const void* g, float* dots,
                          int* status, void* stream) {
  gf::enter();
  if (K % 8 || k > 8) return GFH_BAD_ARG;
  const int wpb = 8;
  int grid = (T + wpb - 1) / wpb;
  const int cap = gf::sm_count() * 4;
  if (grid > cap) grid = cap;
  moe_combine_kernel<<<grid, wpb * 32, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)comb, w, (const __nv_bfloat16*)residual, (__nv_bfloat16*)y, T, k, K, flags, flag_row, epoch,
      world, (const __nv_bfloat16*)g, dots, status);
  return cudaGetLastError() == cudaSuccess ? GFH_OK : GFH_CUDA;
}
