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
  for (int j = s0 + warp; j < s1; j += DEC_WARPS) {
    float kf[PER], vf[PER];
    if (PER == 4) {
      const uint2 ku = *reinterpret_cast<const uint2*>(kb + (long long)j * row_stride);
      const uint2 vu = *reinterpret_cast<const uint2*>(vb + (long long)j * row_stride);
      float2 a = unpack_bf16x2(ku.x), c = unpack_bf16x2(ku.y), d = unpack_bf16x2(vu.x), e = unpack_bf16x2(vu.y);
      kf[0] = a.x; kf[1] = a.y; kf[2] = c.x; kf[3] = c.y;
      vf[0] = d.x; vf[1] = d.y; vf[2] = e.x; vf[3] = e.y;
    } else {
#pragma unroll
      for (int i = 0; i < PER; ++i) {
        kf[i] = __bfloat162float(kb[(long long)j * row_stride + i]);
        vf[i] = __bfloat162float(vb[(long long)j * row_stride + i]);
      }
    }
#pragma unroll
    for (int g = 0; g < DEC_MAX_G; ++g) {
      if (g >= G) break;
      float s = 0.f;
#pragma unroll
      for (int i = 0; i < PER; ++i) s += qv[g][i] * kf[i];
#pragma unroll
      for (int o = 16; o; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
      const float mn = fmaxf(m[g], s);
      const float corr = ex2_approx(m[g] - mn);
      const float p = ex2_approx(s - mn);
      l[g] = l[g] * corr + p;
#pragma unroll
      for (int i = 0; i < PER; ++i) acc[g][i] = acc[g][i] * corr + p * vf[i];
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
    attn_decode_kernel<128><<<grid, DEC_WARPS * 32, 0, st>>>((const __nv_bfloat16*)q, ldq, (const __nv_bfloat16*)kcache,
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
