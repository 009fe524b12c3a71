// Single-query attention over a KV cache (the decode step of generation), grouped-query aware.
//
// The reference decodes by recomputing full attention on the CPU (ghostflow-nn/src/gpt.rs generate loop,
// ghostflow-nn/src/attention.rs:11-49). Here one CTA handles one (sequence, KV head, slice of the cache): its four
// warps stream K and V rows (a warp reads one 256-byte row per load, fully coalesced), every lane owns D / 32
// dimensions, the G = Hq / Hkv query heads that share the KV head are processed together so each cache row is read
// once, and softmax is kept online. Slices are merged by a second kernel. The cache read is the only traffic that
// matters, so the kernel is bandwidth-bound by design; tensor cores would have at most G = 8 useful rows.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "gf_host.h"
#include "gf_ptx.cuh"

namespace gf {

constexpr int DEC_WARPS = 4;
constexpr int DEC_MAX_G = 8;

// q [B, Hq * D] (pitch ldq), k/v cache [B, s_max, Hkv * D]; part_o [B, Hq, splits, D] fp32, part_ml [B, Hq, splits, 2].
template <int D>
__global__ void __launch_bounds__(DEC_WARPS * 32)
attn_decode_kernel(const __nv_bfloat16* __restrict__ q, long long ldq, const __nv_bfloat16* __restrict__ kc,
                   const __nv_bfloat16* __restrict__ vc, long long batch_stride, long long row_stride,
                   const int* __restrict__ lens, int len_all, int Hq, int Hkv, float scale_log2,
                   float* __restrict__ part_o, float* __restrict__ part_ml, int splits) {
  constexpr int PER = D / 32;                 // dimensions per lane
  const int b = blockIdx.x, hk = blockIdx.y, sp = blockIdx.z;
  const int G = Hq / Hkv;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int len = lens ? lens[b] : len_all;
  const int chunk = (len + splits - 1) / splits;
  const int s0 = sp * chunk, s1 = min(len, s0 + chunk);

  float qv[DEC_MAX_G][PER];
  float m[DEC_MAX_G], l[DEC_MAX_G], acc[DEC_MAX_G][PER];
#pragma unroll
  for (int g = 0; g < DEC_MAX_G; ++g) {
    m[g] = -INFINITY;
    l[g] = 0.f;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      acc[g][i] = 0.f;
      qv[g][i] = g < G ? __bfloat162float(q[(long long)b * ldq + (long long)(hk * G + g) * D + lane * PER + i]) * scale_log2
                       : 0.f;
    }
  }
  const __nv_bfloat16* kb = kc + (long long)b * batch_stride + (long long)hk * D + lane * PER;
  const __nv_bfloat16* vb = vc + (long long)b * batch_stride + (long long)hk * D + lane * PER;
  // Four cache rows per warp are in flight at once: the loop is bound by memory latency, not by arithmetic.
  constexpr int UNR = 4;
  for (int j0 = s0 + warp; j0 < s1; j0 += DEC_WARPS * UNR) {
    float kf[UNR][PER], vf[UNR][PER];
#pragma unroll
    for (int u = 0; u < UNR; ++u) {
      const int j = j0 + u * DEC_WARPS;
      if (j < s1) {
        if (PER == 4) {
          const uint2 ku = *reinterpret_cast<const uint2*>(kb + (long long)j * row_stride);
          const uint2 vu = *reinterpret_cast<const uint2*>(vb + (long long)j * row_stride);
          float2 a = unpack_bf16x2(ku.x), c = unpack_bf16x2(ku.y), d = unpack_bf16x2(vu.x), e = unpack_bf16x2(vu.y);
          kf[u][0] = a.x; kf[u][1] = a.y; kf[u][2] = c.x; kf[u][3] = c.y;
          vf[u][0] = d.x; vf[u][1] = d.y; vf[u][2] = e.x; vf[u][3] = e.y;
        } else {
#pragma unroll
          for (int i = 0; i < PER; ++i) {
            kf[u][i] = __bfloat162float(kb[(long long)j * row_stride + i]);
            vf[u][i] = __bfloat162float(vb[(long long)j * row_stride + i]);
          }
        }
      } else {
#pragma unroll
        for (int i = 0; i < PER; ++i) { kf[u][i] = 0.f; vf[u][i] = 0.f; }
      }
    }
#pragma unroll
    for (int g = 0; g < DEC_MAX_G; ++g) {
      if (g >= G) break;
      float sc[UNR];
#pragma unroll
      for (int u = 0; u < UNR; ++u) {
        float t = 0.f;
#pragma unroll
        for (int i = 0; i < PER; ++i) t += qv[g][i] * kf[u][i];
        sc[u] = t;
      }
#pragma unroll
      for (int o = 16; o; o >>= 1) {
#pragma unroll
        for (int u = 0; u < UNR; ++u) sc[u] += __shfl_xor_sync(0xffffffffu, sc[u], o);
      }
      float mn = m[g];
#pragma unroll
      for (int u = 0; u < UNR; ++u) {
        if (j0 + u * DEC_WARPS >= s1) sc[u] = -INFINITY;
        mn = fmaxf(mn, sc[u]);
      }
      if (mn == -INFINITY) continue;
      const float corr = ex2_approx(m[g] - mn);
      float psum = 0.f;
      float pw[UNR];
#pragma unroll
      for (int u = 0; u < UNR; ++u) {
        pw[u] = ex2_approx(sc[u] - mn);
        psum += pw[u];
      }
      l[g] = l[g] * corr + psum;
#pragma unroll
      for (int i = 0; i < PER; ++i) {
        float t = acc[g][i] * corr;
#pragma unroll
        for (int u = 0; u < UNR; ++u) t += pw[u] * vf[u][i];
        acc[g][i] = t;
      }
      m[g] = mn;
    }
  }
  // merge the four warps through shared memory
  __shared__ float sm_m[DEC_WARPS][DEC_MAX_G], sm_l[DEC_WARPS][DEC_MAX_G];
  __shared__ float sm_acc[DEC_WARPS][DEC_MAX_G][D];
  for (int g = 0; g < G; ++g) {
    if (lane == 0) { sm_m[warp][g] = m[g]; sm_l[warp][g] = l[g]; }
#pragma unroll
    for (int i = 0; i < PER; ++i) sm_acc[warp][g][lane * PER + i] = acc[g][i];
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < G * D; idx += blockDim.x) {
    const int g = idx / D, dd = idx % D;
    float mm = -INFINITY;
    for (int w = 0; w < DEC_WARPS; ++w) mm = fmaxf(mm, sm_m[w][g]);
    float ll = 0.f, o = 0.f;
    for (int w = 0; w < DEC_WARPS; ++w) {
      const float c = sm_m[w][g] == -INFINITY ? 0.f : ex2_approx(sm_m[w][g] - mm);
      ll += sm_l[w][g] * c;
      o += sm_acc[w][g][dd] * c;
    }
    const long long base = ((long long)b * Hq + hk * G + g) * splits + sp;
    part_o[base * D + dd] = o;
    if (dd == 0) { part_ml[base * 2] = mm; part_ml[base * 2 + 1] = ll; }
  }
}

// ---------------------------------------------------------------------------------------------------------------
// Tensor-core variant for D = 128: the G <= 8 query heads of a KV group are the (padded) 16 rows of mma.m16n8k16
// tiles, so a cache row costs two MMAs instead of ~160 scalar instructions. A decode step is bound by the cache
// read, for which warp-level MMAs are ample (tcgen05 tiles would need 128 query rows).
//
// Operand fragments come straight from global memory with 16-byte loads, no shared memory:
//  * S = Q K^T contracts over the head dimension, whose order is free. Lane (r = lane / 4, c = lane % 4) loads
//    dims [8c + 32t, 8c + 32t + 8) of "its" row for t = 0..3; register pairs of such a vector are the (b0, b1) /
//    (a0, a2) fragments of two k-steps, the same permutation on both operands.
//  * O = P V contracts over keys (P comes from the S accumulators, the usual register reuse). The B fragment needs
//    two keys of one dim in a register: lanes load dims [16r, 16r + 16) of keys 2c, 2c+1, 8+2c, 9+2c and two PRMTs
//    per register pair transpose them. Column x of output tile j is dim 16x + j.
__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t r;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
  return r;
}

__global__ void __launch_bounds__(DEC_WARPS * 32)
attn_decode_mma_kernel(const __nv_bfloat16* __restrict__ q, long long ldq, const __nv_bfloat16* __restrict__ kc,
                       const __nv_bfloat16* __restrict__ vc, long long batch_stride, long long row_stride,
                       const int* __restrict__ lens, int len_all, int Hq, int Hkv, float scale_log2,
                       float* __restrict__ part_o, float* __restrict__ part_ml, int splits) {
  constexpr int D = 128;
  const int b = blockIdx.x, hk = blockIdx.y, sp = blockIdx.z;
  const int G = Hq / Hkv;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int r = lane >> 2, c = lane & 3;
  const int len = lens ? lens[b] : len_all;
  const int chunk = (len + splits - 1) / splits;
  const int s0 = sp * chunk, s1 = min(len, s0 + chunk);

  uint32_t qa[4][4];
#pragma unroll
  for (int t = 0; t < 4; ++t) {
    uint4 u = make_uint4(0, 0, 0, 0);
    if (r < G) u = *reinterpret_cast<const uint4*>(q + (long long)b * ldq + (long long)(hk * G + r) * D + 8 * c + 32 * t);
    qa[t][0] = u.x; qa[t][1] = u.y; qa[t][2] = u.z; qa[t][3] = u.w;
  }
  float o[16][4];
#pragma unroll
  for (int j = 0; j < 16; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
  float m = -INFINITY, l = 0.f;
  const __nv_bfloat16* kb = kc + (long long)b * batch_stride + (long long)hk * D;
  const __nv_bfloat16* vb = vc + (long long)b * batch_stride + (long long)hk * D;
  const int last = s1 - 1;

  for (int k0 = s0 + warp * 32; k0 < s1; k0 += DEC_WARPS * 32) {
    // ---- S = Q K^T for 32 keys (four tiles of eight)
    uint4 kv[4][4];
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
      const int key = min(k0 + nt * 8 + r, last);
#pragma unroll
      for (int t = 0; t < 4; ++t)
        kv[nt][t] = *reinterpret_cast<const uint4*>(kb + (long long)key * row_stride + 8 * c + 32 * t);
    }
    float sc[4][4];
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
      sc[nt][0] = sc[nt][1] = sc[nt][2] = sc[nt][3] = 0.f;
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        mma_bf16_16816(sc[nt], qa[t][0], 0u, qa[t][1], 0u, kv[nt][t].x, kv[nt][t].y);
        mma_bf16_16816(sc[nt], qa[t][2], 0u, qa[t][3], 0u, kv[nt][t].z, kv[nt][t].w);
      }
    }
    // ---- online softmax on row r (this lane: keys nt * 8 + 2c, + 1 of every tile)
    float mx = -INFINITY;
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int key = k0 + nt * 8 + 2 * c + e;
        sc[nt][e] = key < s1 ? sc[nt][e] * scale_log2 : -INFINITY;
        mx = fmaxf(mx, sc[nt][e]);
      }
    }
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    const float mn = fmaxf(m, mx);           // finite: every block has at least one valid key
    const float corr = ex2_approx(m - mn);
    m = mn;
    uint32_t pa[4];
    float psum = 0.f;
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
      const float p0 = ex2_approx(sc[nt][0] - mn), p1 = ex2_approx(sc[nt][1] - mn);
      psum += p0 + p1;
      pa[nt] = pack_bf16x2(p0, p1);
    }
    l = l * corr + psum;
#pragma unroll
    for (int j = 0; j < 16; ++j) { o[j][0] *= corr; o[j][1] *= corr; }
    // ---- O += P V, two k-steps of 16 keys
#pragma unroll
    for (int ks = 0; ks < 2; ++ks) {
      uint4 vv[4][2];
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) {
        const int key = min(k0 + ks * 16 + (kk >> 1) * 8 + 2 * c + (kk & 1), last);
#pragma unroll
        for (int h = 0; h < 2; ++h)
          vv[kk][h] = *reinterpret_cast<const uint4*>(vb + (long long)key * row_stride + 16 * r + 8 * h);
      }
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const int h = j >> 3, pr = (j & 7) >> 1;
        const uint32_t sel = (j & 1) ? 0x7632u : 0x5410u;
        const uint32_t* w0 = reinterpret_cast<const uint32_t*>(&vv[0][h]);
        const uint32_t* w1 = reinterpret_cast<const uint32_t*>(&vv[1][h]);
        const uint32_t* w2 = reinterpret_cast<const uint32_t*>(&vv[2][h]);
        const uint32_t* w3 = reinterpret_cast<const uint32_t*>(&vv[3][h]);
        mma_bf16_16816(o[j], pa[2 * ks], 0u, pa[2 * ks + 1], 0u, prmt(w0[pr], w1[pr], sel), prmt(w2[pr], w3[pr], sel));
      }
    }
  }
  l += __shfl_xor_sync(0xffffffffu, l, 1);
  l += __shfl_xor_sync(0xffffffffu, l, 2);

  __shared__ float sm_m[DEC_WARPS][DEC_MAX_G], sm_l[DEC_WARPS][DEC_MAX_G];
  __shared__ float sm_acc[DEC_WARPS][DEC_MAX_G][D];
  if (r < G) {
    if (c == 0) { sm_m[warp][r] = m; sm_l[warp][r] = l; }
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      sm_acc[warp][r][(2 * c) * 16 + j] = o[j][0];
      sm_acc[warp][r][(2 * c + 1) * 16 + j] = o[j][1];
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < G * D; idx += blockDim.x) {
    const int g = idx / D, dd = idx % D;
    float mm = -INFINITY;
    for (int w = 0; w < DEC_WARPS; ++w) mm = fmaxf(mm, sm_m[w][g]);
    float ll = 0.f, ov = 0.f;
    for (int w = 0; w < DEC_WARPS; ++w) {
      const float cw = sm_m[w][g] == -INFINITY ? 0.f : ex2_approx(sm_m[w][g] - mm);
      ll += sm_l[w][g] * cw;
      ov += sm_acc[w][g][dd] * cw;
    }
    const long long base = ((long long)b * Hq + hk * G + g) * splits + sp;
    part_o[base * D + dd] = ov;
    if (dd == 0) { part_ml[base * 2] = mm; part_ml[base * 2 + 1] = ll; }
  }
}

template <int D>
__global__ void attn_decode_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                         __nv_bfloat16* __restrict__ out, long long ldo, int Hq, int splits) {
  const int b = blockIdx.x, h = blockIdx.y, dd = threadIdx.x;
  const long long base = ((long long)b * Hq + h) * splits;
  float mm = -INFINITY;
  for (int s = 0; s < splits; ++s) mm = fmaxf(mm, part_ml[(base + s) * 2]);
  float ll = 0.f, o = 0.f;
  for (int s = 0; s < splits; ++s) {
    const float ms = part_ml[(base + s) * 2];
    const float c = ms == -INFINITY ? 0.f : ex2_approx(ms - mm);
    ll += part_ml[(base + s) * 2 + 1] * c;
    o += part_o[(base + s) * D + dd] * c;
  }
  out[(long long)b * ldo + (long long)h * D + dd] = __float2bfloat16(ll > 0.f ? o / ll : 0.f);
}

}  // namespace gf

using namespace gf;

// q [B, Hq * D] pitch ldq; caches [B, s_max, Hkv * D] contiguous; out [B, Hq * D] pitch ldo.
// `lens` (device int[B]) gives the valid length per sequence; nullptr: `len_all` for every sequence.
// scratch: fp32 [B * Hq * splits * (D + 2)].
GF_API int gf_attn_decode(const void* q, long long ldq, const void* kcache, const void* vcache, int s_max,
                          const int* lens, int len_all, void* out, long long ldo, int B, int Hq, int Hkv, int D,
                          float scale, int splits, float* scratch, void* stream) {
  gf::enter();
  if (B <= 0 || Hq % Hkv || Hq / Hkv > DEC_MAX_G || (D != 64 && D != 128) || splits < 1 || !scratch) return GFH_BAD_ARG;
  float* part_o = scratch;
  float* part_ml = scratch + (long long)B * Hq * splits * D;
  const long long row = (long long)Hkv * D, batch = (long long)s_max * row;
  const float sl2 = scale * 1.4426950408889634f;
  dim3 grid(B, Hkv, splits);
  cudaStream_t st = (cudaStream_t)stream;
  if (D == 128) {
    // warps that get no key block leave m = -inf, l = 0 and are ignored by the merge
    attn_decode_mma_kernel<<<grid, DEC_WARPS * 32, 0, st>>>((const __nv_bfloat16*)q, ldq, (const __nv_bfloat16*)kcache,
                                                           (const __nv_bfloat16*)vcache, batch, row, lens, len_all, Hq,
                                                           Hkv, sl2, part_o, part_ml, splits);
    attn_decode_merge_kernel<128><<<dim3(B, Hq), 128, 0, st>>>(part_o, part_ml, (__nv_bfloat16*)out, ldo, Hq, splits);
  } else {
    attn_decode_kernel<64><<<grid, DEC_WARPS * 32, 0, st>>>((const __nv_bfloat16*)q, ldq, (const __nv_bfloat16*)kcache,
                                                           (const __nv_bfloat16*)vcache, batch, row, lens, len_all, Hq,
                                                           Hkv, sl2, part_o, part_ml, splits);
    attn_decode_merge_kernel<64><<<dim3(B, Hq), 64, 0, st>>>(part_o, part_ml, (__nv_bfloat16*)out, ldo, Hq, splits);
  }
  gf::note_extra_launches(1);
  return cudaGetLastError() == cudaSuccess ? GFH_OK : GFH_CUDA;
}
