// RMSNorm and LayerNorm, forward and backward, bf16 in/out with fp32 arithmetic.
//
// One CTA per row keeps the row in registers (16-byte loads), so each tensor is read
// once and written once. The weight/bias gradients are cross-row sums: each CTA of a
// persistent grid accumulates its rows in registers, writes one partial row to a scratch
// buffer, and a second small kernel folds the partials.
//
// Formulas follow the reference's CPU code: RMSNorm x / sqrt(mean(x^2) + eps) * w
// (ghostflow-nn/src/llama.rs:154-185); LayerNorm with biased variance
// (ghostflow-nn/src/norm.rs:239-270). The reference only names GPU kernels for these
// (ghostflow-cuda/src/kernels/mod.rs:103-106) without implementing them.
#include "gf_host.h"
#include "gf_ptx.cuh"

namespace gf {

constexpr int NORM_THREADS = 256;
constexpr int NORM_MAXV = 4;  // 16-byte vectors per thread kept in registers -> D <= 8192

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  __syncthreads();
  if (l == 0) red[w] = v;
  __syncthreads();
  float t = (l < (blockDim.x >> 5)) ? red[l] : 0.f;
  t = warp_sum(t);
  return t;
}

__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&f)[8]) {
  uint4 u = *reinterpret_cast<const uint4*>(p);
  float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float (&f)[8]) {
  uint4 u;
  u.x = pack_bf16x2(f[0], f[1]); u.y = pack_bf16x2(f[2], f[3]);
  u.z = pack_bf16x2(f[4], f[5]); u.w = pack_bf16x2(f[6], f[7]);
  *reinterpret_cast<uint4*>(p) = u;
}

// ------------------------------------------------------------------ RMSNorm forward
// Optional fused residual add: h = x + res is written to `h_out` and normalised.
__global__ void __launch_bounds__(NORM_THREADS)
rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ res,
                   const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ y,
                   __nv_bfloat16* __restrict__ h_out, float* __restrict__ rstd_out, int T, int D, float eps) {
  __shared__ float red[32];
  const int nv = D >> 3;
  for (int row = blockIdx.x; row < T; row += gridDim.x) {
    const __nv_bfloat16* xr = x + (long long)row * D;
    float xv[NORM_MAXV][8];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < NORM_MAXV; ++i) {
      const int v = threadIdx.x + i * NORM_THREADS;
      if (v < nv) {
        load8(xr + v * 8, xv[i]);
        if (res) {
          float rv[8];
          load8(res + (long long)row * D + v * 8, rv);
#pragma unroll
          for (int j = 0; j < 8; ++j) xv[i][j] += rv[j];
          if (h_out) {
            store8(h_out + (long long)row * D + v * 8, xv[i]);
            // normalise exactly what was stored (bf16-rounded) so backward sees the same h
            load8(h_out + (long long)row * D + v * 8, xv[i]);
          }
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) ss += xv[i][j] * xv[i][j];
      }
    }
    ss = block_sum(ss, red);
    const float rstd = rsqrtf(ss / (float)D + eps);
    if (threadIdx.x == 0 && rstd_out) rstd_out[row] = rstd;
#pragma unroll
    for (int i = 0; i < NORM_MAXV; ++i) {
      const int v = threadIdx.x + i * NORM_THREADS;
      if (v < nv) {
        float wv[8], o[8];
        load8(w + v * 8, wv);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = xv[i][j] * rstd * wv[j];
        store8(y + (long long)row * D + v * 8, o);
      }
    }
  }
}

// ------------------------------------------------------------------ RMSNorm backward
// dx = rstd * g - x * rstd^3 * mean(g * x), g = dy * w ; dw partial = sum_rows dy * x * rstd.
// If `dres` is given, it is added into dx (gradient arriving through the residual branch).
// Operands stay packed (bf16x8 in a uint4) between the two passes over a row and only the dw accumulators are
// fp32, so for D <= 4096 (MAXV = 2) a thread needs about 64 registers and four CTAs fit on an SM.
__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
  float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}

template <int MAXV>
__global__ void __launch_bounds__(NORM_THREADS, MAXV == 1 ? 4 : (MAXV == 2 ? 3 : 2))
rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                   const __nv_bfloat16* __restrict__ dy, const float* __restrict__ rstd_in,
                   const __nv_bfloat16* __restrict__ dres, __nv_bfloat16* __restrict__ dx,
                   float* __restrict__ dw_partial, int T, int D) {
  __shared__ float red[32];
  const int nv = D >> 3;
  float dwacc[MAXV][8];
  uint4 wp[MAXV];
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int v = threadIdx.x + i * NORM_THREADS;
#pragma unroll
    for (int j = 0; j < 8; ++j) dwacc[i][j] = 0.f;
    wp[i] = (v < nv) ? *reinterpret_cast<const uint4*>(w + v * 8) : make_uint4(0, 0, 0, 0);
  }
  for (int row = blockIdx.x; row < T; row += gridDim.x) {
    const float rstd = rstd_in[row];
    uint4 xp[MAXV], gp[MAXV], rp[MAXV];
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
      const int v = threadIdx.x + i * NORM_THREADS;
      if (v < nv) {
        xp[i] = *reinterpret_cast<const uint4*>(x + (long long)row * D + v * 8);
        gp[i] = *reinterpret_cast<const uint4*>(dy + (long long)row * D + v * 8);
        if (dres) rp[i] = *reinterpret_cast<const uint4*>(dres + (long long)row * D + v * 8);
      }
    }
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
      const int v = threadIdx.x + i * NORM_THREADS;
      if (v < nv) {
        float xv[8], gv[8], wv[8];
        unpack8(xp[i], xv); unpack8(gp[i], gv); unpack8(wp[i], wv);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          dwacc[i][j] += gv[j] * xv[j] * rstd;
          dot += gv[j] * wv[j] * xv[j];
        }
      }
    }
    dot = block_sum(dot, red);
    const float c = dot * rstd * rstd * rstd / (float)D;
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
      const int v = threadIdx.x + i * NORM_THREADS;
      if (v < nv) {
        float xv[8], gv[8], wv[8], o[8];
        unpack8(xp[i], xv); unpack8(gp[i], gv); unpack8(wp[i], wv);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = rstd * gv[j] * wv[j] - c * xv[j];
        if (dres) {
          float rv[8];
          unpack8(rp[i], rv);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] += rv[j];
        }
        store8(dx + (long long)row * D + v * 8, o);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int v = threadIdx.x + i * NORM_THREADS;
    if (v < nv) {
      float* dst = dw_partial + (long long)blockIdx.x * D + v * 8;
      *reinterpret_cast<float4*>(dst) = make_float4(dwacc[i][0], dwacc[i][1], dwacc[i][2], dwacc[i][3]);
      *reinterpret_cast<float4*>(dst + 4) = make_float4(dwacc[i][4], dwacc[i][5], dwacc[i][6], dwacc[i][7]);
    }
  }
}

// Fold `nparts` partial rows of length D; writes bf16 (optionally accumulating into existing bf16).
// One CTA per 32 columns: its eight warps stride over the partial rows (each warp reads 128 contiguous bytes per
// row), then the eight per-warp sums are combined through shared memory. With hundreds of partial rows this keeps
// 4096 / 32 = 128 CTAs busy instead of 16 threads-per-column chains.
__global__ void __launch_bounds__(256)
fold_partials_kernel(const float* __restrict__ partial, __nv_bfloat16* __restrict__ out, int nparts, int D,
                     int accumulate) {
  __shared__ float sm[8][32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int d = blockIdx.x * 32 + lane;
  float s = 0.f;
  if (d < D)
    for (int p = warp; p < nparts; p += 8) s += partial[(long long)p * D + d];
  sm[warp][lane] = s;
  __syncthreads();
  if (warp == 0 && d < D) {
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) t += sm[w][lane];
    if (accumulate) t += __bfloat162float(out[d]);
    out[d] = __float2bfloat16(t);
  }
}

// ------------------------------------------------------------------ LayerNorm forward
__global__ void __launch_bounds__(NORM_THREADS)
layernorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                     const __nv_bfloat16* __restrict__ b, __nv_bfloat16* __restrict__ y, float* __restrict__ mean_out,
                     float* __restrict__ rstd_out, int T, int D, float eps) {
  __shared__ float red[32];
  const int nv = D >> 3;
  for (int row = blockIdx.x; row < T; row += gridDim.x) {
    float xv[NORM_MAXV][8];
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < NORM_MAXV; ++i) {
      const int v = threadIdx.x + i * NORM_THREADS;
      if (v < nv) {
        load8(x + (long long)row * D + v * 8, xv[i]);
#pragma unroll
        for (int j = 0; j < 8; ++j) s += xv[i][j];
      }
    }
    const float mean = block_sum(s, red) / (float)D;
    float sq = 0.f;
#pragma unroll
    for (int i = 0; i < NORM_MAXV; ++i) {
      const int v = threadIdx.x + i * NORM_THREADS;
      if (v < nv) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float d = xv[i][j] - mean;
          sq += d * d;
        }
      }
    }
    const float var = block_sum(sq, red) / (float)D;
    const float rstd = rsqrtf(var + eps);
    if (threadIdx.x == 0) {
      if (mean_out) mean_out[row] = mean;
      if (rstd_out) rstd_out[row] = rstd;
    }
#pragma unroll
    for (int i = 0; i < NORM_MAXV; ++i) {
      const int v = threadIdx.x + i * NORM_THREADS;
      if (v < nv) {
        float wv[8], bv[8], o[8];
        load8(w + v * 8, wv);
        if (b) load8(b + v * 8, bv);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = (xv[i][j] - mean) * rstd * wv[j] + (b ? bv[j] : 0.f);
        store8(y + (long long)row * D + v * 8, o);
      }
    }
  }
}

// ------------------------------------------------------------------ LayerNorm backward
// xhat = (x - mean) * rstd ; g = dy * w ; dx = rstd * (g - mean(g) - xhat * mean(g * xhat))
__global__ void __launch_bounds__(NORM_THREADS)
layernorm_bwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                     const __nv_bfloat16* __restrict__ dy, const float* __restrict__ mean_in,
                     const float* __restrict__ rstd_in, __nv_bfloat16* __restrict__ dx,
                     float* __restrict__ dw_partial, float* __restrict__ db_partial, int T, int D) {
  __shared__ float red[32];
  const int nv = D >> 3;
  float dwacc[NORM_MAXV][8], dbacc[NORM_MAXV][8], wv[NORM_MAXV][8];
#pragma unroll
  for (int i = 0; i < NORM_MAXV; ++i) {
    const int v = threadIdx.x + i * NORM_THREADS;
#pragma unroll
    for (int j = 0; j < 8; ++j) dwacc[i][j] = dbacc[i][j] = 0.f;
    if (v < nv) load8(w + v * 8, wv[i]);
  }
  for (int row = blockIdx.x; row < T; row += gridDim.x) {
    const float mean = mean_in[row], rstd = rstd_in[row];
    float xh[NORM_MAXV][8], gv[NORM_MAXV][8];
    float sg = 0.f, sgx = 0.f;
#pragma unroll
    for (int i = 0; i < NORM_MAXV; ++i) {
      const int v = threadIdx.x + i * NORM_THREADS;
      if (v < nv) {
        load8(x + (long long)row * D + v * 8, xh[i]);
        load8(dy + (long long)row * D + v * 8, gv[i]);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          xh[i][j] = (xh[i][j] - mean) * rstd;
          dwacc[i][j] += gv[i][j] * xh[i][j];
          dbacc[i][j] += gv[i][j];
          gv[i][j] *= wv[i][j];
          sg += gv[i][j];
          sgx += gv[i][j] * xh[i][j];
        }
      }
    }
    sg = block_sum(sg, red) / (float)D;
    sgx = block_sum(sgx, red) / (float)D;
#pragma unroll
    for (int i = 0; i < NORM_MAXV; ++i) {
      const int v = threadIdx.x + i * NORM_THREADS;
      if (v < nv) {
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = rstd * (gv[i][j] - sg - xh[i][j] * sgx);
        store8(dx + (long long)row * D + v * 8, o);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < NORM_MAXV; ++i) {
    const int v = threadIdx.x + i * NORM_THREADS;
    if (v < nv) {
      float* dst = dw_partial + (long long)blockIdx.x * D + v * 8;
      float* dsb = db_partial + (long long)blockIdx.x * D + v * 8;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        dst[j] = dwacc[i][j];
        dsb[j] = dbacc[i][j];
      }
    }
  }
}


// ------------------------------------------------------------------ LayerNorm for short rows (D <= 1024)
// With D = 768 a 256-thread CTA per row leaves 160 threads idle and pays two block-wide reductions per row. Here
// one WARP owns a row (VPL 16-byte vectors per lane), the sums are warp shuffles, and a CTA has eight rows in
// flight. In the backward pass every lane keeps its slice of the weight / bias gradient in registers over all its
// rows; the eight warps of a CTA then add their slices in shared memory and the CTA writes one partial row.
template <int VPL>
__global__ void __launch_bounds__(NORM_THREADS)
layernorm_fwd_warp_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                          const __nv_bfloat16* __restrict__ b, __nv_bfloat16* __restrict__ y,
                          float* __restrict__ mean_out, float* __restrict__ rstd_out, int T, int D, float eps) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nv = D >> 3;
  constexpr int WPC = NORM_THREADS / 32;
  float wv[VPL][8], bv[VPL][8];
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    const int v = lane + i * 32;
#pragma unroll
    for (int j = 0; j < 8; ++j) bv[i][j] = 0.f;
    if (v < nv) {
      load8(w + v * 8, wv[i]);
      if (b) load8(b + v * 8, bv[i]);
    }
  }
  for (int row = blockIdx.x * WPC + warp; row < T; row += gridDim.x * WPC) {
    float xv[VPL][8];
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      const int v = lane + i * 32;
      if (v < nv) {
        load8(x + (long long)row * D + v * 8, xv[i]);
#pragma unroll
        for (int j = 0; j < 8; ++j) s += xv[i][j];
      }
    }
    const float mean = warp_sum(s) / (float)D;
    float sq = 0.f;
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      if (lane + i * 32 < nv) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float d = xv[i][j] - mean;
          sq += d * d;
        }
      }
    }
    const float rstd = rsqrtf(warp_sum(sq) / (float)D + eps);
    if (lane == 0) {
      if (mean_out) mean_out[row] = mean;
      if (rstd_out) rstd_out[row] = rstd;
    }
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      const int v = lane + i * 32;
      if (v < nv) {
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = (xv[i][j] - mean) * rstd * wv[i][j] + bv[i][j];
        store8(y + (long long)row * D + v * 8, o);
      }
    }
  }
}

template <int VPL>
__global__ void __launch_bounds__(NORM_THREADS, 2)
layernorm_bwd_warp_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                          const __nv_bfloat16* __restrict__ dy, const float* __restrict__ mean_in,
                          const float* __restrict__ rstd_in, __nv_bfloat16* __restrict__ dx,
                          float* __restrict__ dw_partial, float* __restrict__ db_partial, int T, int D) {
  __shared__ float acc[2][1024];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nv = D >> 3;
  constexpr int WPC = NORM_THREADS / 32;
  for (int i = threadIdx.x; i < D; i += NORM_THREADS) acc[0][i] = acc[1][i] = 0.f;
  // the weight is re-read for every row (1.5 KB, served by L1): keeping it in registers next to the two
  // accumulators would push the kernel to one CTA per SM
  float dwacc[VPL][8], dbacc[VPL][8];
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
#pragma unroll
    for (int j = 0; j < 8; ++j) dwacc[i][j] = dbacc[i][j] = 0.f;
  }
  for (int row = blockIdx.x * WPC + warp; row < T; row += gridDim.x * WPC) {
    const float mean = mean_in[row], rstd = rstd_in[row];
    float xh[VPL][8], gv[VPL][8];
    float sg = 0.f, sgx = 0.f;
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      const int v = lane + i * 32;
      if (v < nv) {
        float wv[8];
        load8(x + (long long)row * D + v * 8, xh[i]);
        load8(dy + (long long)row * D + v * 8, gv[i]);
        load8(w + v * 8, wv);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          xh[i][j] = (xh[i][j] - mean) * rstd;
          dwacc[i][j] += gv[i][j] * xh[i][j];
          dbacc[i][j] += gv[i][j];
          gv[i][j] *= wv[j];
          sg += gv[i][j];
          sgx += gv[i][j] * xh[i][j];
        }
      }
    }
    sg = warp_sum(sg) / (float)D;
    sgx = warp_sum(sgx) / (float)D;
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      const int v = lane + i * 32;
      if (v < nv) {
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = rstd * (gv[i][j] - sg - xh[i][j] * sgx);
        store8(dx + (long long)row * D + v * 8, o);
      }
    }
  }
  __syncthreads();
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    const int v = lane + i * 32;
    if (v < nv) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        atomicAdd(&acc[0][v * 8 + j], dwacc[i][j]);
        atomicAdd(&acc[1][v * 8 + j], dbacc[i][j]);
      }
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < D; i += NORM_THREADS) {
    dw_partial[(long long)blockIdx.x * D + i] = acc[0][i];
    db_partial[(long long)blockIdx.x * D + i] = acc[1][i];
  }
}

// ------------------------------------------------------------------ column sums (bias gradients)
// out[d] = sum over rows of x[row, d]: every CTA of a persistent grid adds its rows in registers (fp32) and writes
// one partial row; fold_partials_kernel adds the partial rows. x is read once, 16 bytes per thread and step.
template <int VPT>
__global__ void __launch_bounds__(NORM_THREADS)
colsum_partial_kernel(const __nv_bfloat16* __restrict__ x, long long ld, float* __restrict__ partial, int T, int D) {
  const int nv = D >> 3;
  float acc[VPT][8];
#pragma unroll
  for (int i = 0; i < VPT; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;
  for (int row = blockIdx.x; row < T; row += gridDim.x) {
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int v = threadIdx.x + i * NORM_THREADS;
      if (v < nv) {
        float f[8];
        load8(x + (long long)row * ld + v * 8, f);
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] += f[j];
      }
    }
  }
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = threadIdx.x + i * NORM_THREADS;
    if (v < nv) {
      float* dst = partial + (long long)blockIdx.x * D + v * 8;
#pragma unroll
      for (int j = 0; j < 8; ++j) dst[j] = acc[i][j];
    }
  }
}

static inline int norm_grid(int T) {
  int g = sm_count() * 4;
  return T < g ? T : g;
}

}  // namespace gf

using namespace gf;

GF_API int gf_norm_bwd_grid(int T) { return norm_grid(T); }

GF_API int gf_rmsnorm_fwd(const void* x, const void* res, const void* w, void* y, void* h_out, float* rstd, int T,
                          int D, float eps, void* stream) {
  gf::enter();
  if (D % 8 || D > NORM_THREADS * NORM_MAXV * 8 || T <= 0) return GFH_BAD_ARG;
  rmsnorm_fwd_kernel<<<T, NORM_THREADS, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)x, (const __nv_bfloat16*)res, (const __nv_bfloat16*)w, (__nv_bfloat16*)y,
      (__nv_bfloat16*)h_out, rstd, T, D, eps);
  return cudaGetLastError() == cudaSuccess ? GFH_OK : GFH_CUDA;
}

// scratch: fp32 [gf_norm_bwd_grid(T), D]. dw is bf16 [D]; accumulate=1 adds into it.
GF_API int gf_rmsnorm_bwd(const void* x, const void* w, const void* dy, const float* rstd, const void* dres,
                          void* dx, void* dw, float* scratch, int T, int D, int accumulate, void* stream) {
  gf::enter();
  if (D % 8 || D > NORM_THREADS * NORM_MAXV * 8 || T <= 0) return GFH_BAD_ARG;
  const int g = norm_grid(T);
  auto kern = D <= NORM_THREADS * 8 ? rmsnorm_bwd_kernel<1>
              : D <= NORM_THREADS * 16 ? rmsnorm_bwd_kernel<2> : rmsnorm_bwd_kernel<NORM_MAXV>;
  kern<<<g, NORM_THREADS, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, (const __nv_bfloat16*)dy, rstd, (const __nv_bfloat16*)dres,
      (__nv_bfloat16*)dx, scratch, T, D);
  fold_partials_kernel<<<(D + 31) / 32, 256, 0, (cudaStream_t)stream>>>(scratch, (__nv_bfloat16*)dw, g, D,
                                                                          accumulate);
  gf::note_extra_launches(1);
  return cudaGetLastError() == cudaSuccess ? GFH_OK : GFH_CUDA;
}

// x: bf16 [T, D] with row pitch ld (elements, multiple of 8); out: bf16 [D]; scratch: fp32 [gf_norm_bwd_grid(T), D].
GF_API int gf_colsum_bf16(const void* x, long long ld, void* out, float* scratch, int T, int D, int accumulate,
                          void* stream) {
  gf::enter();
  if (D % 8 || ld % 8 || ld < D || D > NORM_THREADS * NORM_MAXV * 8 || T <= 0 || !scratch) return GFH_BAD_ARG;
  const int g = norm_grid(T);
  auto kern = D <= NORM_THREADS * 8 ? colsum_partial_kernel<1>
              : D <= NORM_THREADS * 16 ? colsum_partial_kernel<2> : colsum_partial_kernel<NORM_MAXV>;
  kern<<<g, NORM_THREADS, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)x, ld, scratch, T, D);
  fold_partials_kernel<<<(D + 31) / 32, 256, 0, (cudaStream_t)stream>>>(scratch, (__nv_bfloat16*)out, g, D,
                                                                          accumulate);
  gf::note_extra_launches(1);
  return cudaGetLastError() == cudaSuccess ? GFH_OK : GFH_CUDA;
}

GF_API int gf_layernorm_fwd(const void* x, const void* w, const void* b, void* y, float* mean, float* rstd, int T,
                            int D, float eps, void* stream) {
  gf::enter();
  if (D % 8 || D > NORM_THREADS * NORM_MAXV * 8 || T <= 0) return GFH_BAD_ARG;
  if (D <= 1024) {   // one warp per row
    const int vpl = (D / 8 + 31) / 32;
    auto kern = vpl == 1 ? layernorm_fwd_warp_kernel<1> : vpl == 2 ? layernorm_fwd_warp_kernel<2>
                : vpl == 3 ? layernorm_fwd_warp_kernel<3> : layernorm_fwd_warp_kernel<4>;
    const int want = (T + 7) / 8, cap = sm_count() * 8;
    kern<<<want < cap ? want : cap, NORM_THREADS, 0, (cudaStream_t)stream>>>(
        (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, (const __nv_bfloat16*)b, (__nv_bfloat16*)y, mean, rstd, T,
        D, eps);
    return cudaGetLastError() == cudaSuccess ? GFH_OK : GFH_CUDA;
  }
  layernorm_fwd_kernel<<<T, NORM_THREADS, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, (const __nv_bfloat16*)b, (__nv_bfloat16*)y, mean, rstd, T,
      D, eps);
  return cudaGetLastError() == cudaSuccess ? GFH_OK : GFH_CUDA;
}

// scratch: fp32 [2, gf_norm_bwd_grid(T), D]
GF_API int gf_layernorm_bwd(const void* x, const void* w, const void* dy, const float* mean, const float* rstd,
                            void* dx, void* dw, void* db, float* scratch, int T, int D, int accumulate,
                            void* stream) {
  gf::enter();
  if (D % 8 || D > NORM_THREADS * NORM_MAXV * 8 || T <= 0) return GFH_BAD_ARG;
  const int g = norm_grid(T);
  float* s2 = scratch + (long long)g * D;
  if (D <= 1024) {   // one warp per row; the CTA still writes one partial row per gradient
    const int vpl = (D / 8 + 31) / 32;
    auto kern = vpl == 1 ? layernorm_bwd_warp_kernel<1> : vpl == 2 ? layernorm_bwd_warp_kernel<2>
                : vpl == 3 ? layernorm_bwd_warp_kernel<3> : layernorm_bwd_warp_kernel<4>;
    kern<<<g, NORM_THREADS, 0, (cudaStream_t)stream>>>(
        (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, (const __nv_bfloat16*)dy, mean, rstd, (__nv_bfloat16*)dx,
        scratch, s2, T, D);
  } else
  layernorm_bwd_kernel<<<g, NORM_THREADS, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, (const __nv_bfloat16*)dy, mean, rstd, (__nv_bfloat16*)dx,
      scratch, s2, T, D);
  fold_partials_kernel<<<(D + 31) / 32, 256, 0, (cudaStream_t)stream>>>(scratch, (__nv_bfloat16*)dw, g, D,
                                                                          accumulate);
  gf::note_extra_launches(db ? 2 : 1);
  if (db)
    fold_partials_kernel<<<(D + 31) / 32, 256, 0, (cudaStream_t)stream>>>(s2, (__nv_bfloat16*)db, g, D,
                                                                            accumulate);
  return cudaGetLastError() == cudaSuccess ? GFH_OK : GFH_CUDA;
}
