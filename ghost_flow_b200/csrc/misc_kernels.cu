// Smaller CUDA kernels off the transformer hot path (fp32 I/O):
//   * NeRF positional encoding and the volume-rendering compositor (one ray per thread, early termination
//     once transmittance is negligible) - ghostflow-nn/src/nerf.rs:111-147, 353-408 (CPU loops there)
//   * farthest-point sampling and k-nearest-neighbour grouping for point clouds, per-face mesh normals -
//     ghostflow-nn/src/point_cloud.rs:326-470, mesh.rs:55-113
//   * INT8 quantise / dequantise / fake-quantise, per tensor or per channel, symmetric or asymmetric -
//     ghostflow-nn/src/quantization.rs:77-240
//   * inference Conv2d + BatchNorm + ReLU in one pass (direct convolution, NCHW, any output width) and
//     BatchNorm statistics / normalisation - ghostflow-cuda/src/optimized_kernels.cu:125-179 (limited to
//     out_w <= 32, no bias), ghostflow-nn/src/norm.rs:39-201
#include "gf_host.h"
#include "gf_ptx.cuh"

namespace gf {

// ------------------------------------------------------------------ NeRF
// x [n, d] -> out [n, d * (2F + include)]: per input dim: [x,] sin(2^0 x), cos(2^0 x), sin(2^1 x), ...
__global__ void posenc_kernel(const float* __restrict__ x, float* __restrict__ out, long long n, int d, int F,
                              int include) {
  const int per = 2 * F + include;
  const long long total = n * d;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const float v = x[i];
    float* o = out + i * per;
    int k = 0;
    if (include) o[k++] = v;
    float f = 1.f;
    for (int j = 0; j < F; ++j) {
      float s, c;
      sincosf(v * f, &s, &c);
      o[k++] = s;
      o[k++] = c;
      f *= 2.f;
    }
  }
}

// rgb [R,S,3], sigma [R,S], z [R,S], ray_norm [R] (or null) -> color [R,3], depth [R], acc [R], weights [R,S]
__global__ void volume_render_kernel(const float* __restrict__ rgb, const float* __restrict__ sigma,
                                     const float* __restrict__ z, const float* __restrict__ ray_norm,
                                     float* __restrict__ color, float* __restrict__ depth, float* __restrict__ acc,
                                     float* __restrict__ weights, int R, int S, int white_bg) {
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= R) return;
  const float* zr = z + (long long)r * S;
  const float* sr = sigma + (long long)r * S;
  const float* cr = rgb + (long long)r * S * 3;
  float* wr = weights + (long long)r * S;
  const float nrm = ray_norm ? ray_norm[r] : 1.f;
  float T = 1.f, c0 = 0.f, c1 = 0.f, c2 = 0.f, dsum = 0.f, asum = 0.f;
  int i = 0;
  for (; i < S; ++i) {
    const float delta = (i + 1 < S ? zr[i + 1] - zr[i] : 1e10f) * nrm;
    const float alpha = 1.f - __expf(-sr[i] * delta);
    const float w = T * alpha;
    wr[i] = w;
    c0 += w * cr[i * 3 + 0];
    c1 += w * cr[i * 3 + 1];
    c2 += w * cr[i * 3 + 2];
    dsum += w * zr[i];
    asum += w;
    T *= 1.f - alpha + 1e-10f;
    if (T < 1e-6f) {  // nothing behind this sample can contribute
      ++i;
      break;
    }
  }
  for (; i < S; ++i) wr[i] = 0.f;
  if (white_bg) {
    c0 += 1.f - asum; c1 += 1.f - asum; c2 += 1.f - asum;
  }
  color[r * 3 + 0] = c0; color[r * 3 + 1] = c1; color[r * 3 + 2] = c2;
  depth[r] = dsum;
  acc[r] = asum;
}

// ------------------------------------------------------------------ point clouds
// One block per batch element. pts [B,N,3] -> idx [B,M]; dist is scratch [B,N].
__global__ void fps_kernel(const float* __restrict__ pts, int* __restrict__ idx, float* __restrict__ dist, int N,
                           int M, int start) {
  __shared__ float sval[32];
  __shared__ int sidx[32];
  __shared__ int cur;
  const int b = blockIdx.x;
  const float* p = pts + (long long)b * N * 3;
  float* d = dist + (long long)b * N;
  for (int i = threadIdx.x; i < N; i += blockDim.x) d[i] = 1e30f;
  if (threadIdx.x == 0) {
    cur = start % N;
    idx[(long long)b * M] = cur;
  }
  __syncthreads();
  for (int m = 1; m < M; ++m) {
    const float cx = p[cur * 3], cy = p[cur * 3 + 1], cz = p[cur * 3 + 2];
    float best = -1.f;
    int bi = 0;
    for (int i = threadIdx.x; i < N; i += blockDim.x) {
      const float dx = p[i * 3] - cx, dy = p[i * 3 + 1] - cy, dz = p[i * 3 + 2] - cz;
      const float nd = fminf(d[i], dx * dx + dy * dy + dz * dz);
      d[i] = nd;
      if (nd > best) { best = nd; bi = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
    }
    if ((threadIdx.x & 31) == 0) { sval[threadIdx.x >> 5] = best; sidx[threadIdx.x >> 5] = bi; }
    __syncthreads();
    if (threadIdx.x == 0) {
      float bb = sval[0];
      int ii = sidx[0];
      for (int w = 1; w < (blockDim.x >> 5); ++w)
        if (sval[w] > bb || (sval[w] == bb && sidx[w] < ii)) { bb = sval[w]; ii = sidx[w]; }
      cur = ii;
      idx[(long long)b * M + m] = ii;
    }
    __syncthreads();
  }
}

// One thread per query: the K nearest points (insertion into a small sorted list; K <= 64).
__global__ void knn_kernel(const float* __restrict__ pts, const float* __restrict__ queries, int* __restrict__ out,
                           int B, int N, int Q, int K) {
  const long long g = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (g >= (long long)B * Q) return;
  const int b = (int)(g / Q);
  const float* p = pts + (long long)b * N * 3;
  const float qx = queries[g * 3], qy = queries[g * 3 + 1], qz = queries[g * 3 + 2];
  float bd[64];
  int bi[64];
  for (int k = 0; k < K; ++k) { bd[k] = 1e30f; bi[k] = 0; }
  for (int i = 0; i < N; ++i) {
    const float dx = p[i * 3] - qx, dy = p[i * 3 + 1] - qy, dz = p[i * 3 + 2] - qz;
    const float d = dx * dx + dy * dy + dz * dz;
    if (d < bd[K - 1]) {
      int k = K - 1;
      while (k > 0 && bd[k - 1] > d) { bd[k] = bd[k - 1]; bi[k] = bi[k - 1]; --k; }
      bd[k] = d;
      bi[k] = i;
    }
  }
  for (int k = 0; k < K; ++k) out[g * K + k] = bi[k];
}

// verts [V,3], faces [F,3] (int) -> normals [F,3] (unit), areas [F]
__global__ void face_normals_kernel(const float* __restrict__ verts, const int* __restrict__ faces,
                                    float* __restrict__ normals, float* __restrict__ areas, int F) {
  const int f = blockIdx.x * blockDim.x + threadIdx.x;
  if (f >= F) return;
  const int a = faces[f * 3], b = faces[f * 3 + 1], c = faces[f * 3 + 2];
  const float ux = verts[b * 3] - verts[a * 3], uy = verts[b * 3 + 1] - verts[a * 3 + 1], uz = verts[b * 3 + 2] - verts[a * 3 + 2];
  const float vx = verts[c * 3] - verts[a * 3], vy = verts[c * 3 + 1] - verts[a * 3 + 1], vz = verts[c * 3 + 2] - verts[a * 3 + 2];
  const float nx = uy * vz - uz * vy, ny = uz * vx - ux * vz, nz = ux * vy - uy * vx;
  const float len = sqrtf(nx * nx + ny * ny + nz * nz);
  const float inv = len > 1e-20f ? 1.f / len : 0.f;
  normals[f * 3] = nx * inv; normals[f * 3 + 1] = ny * inv; normals[f * 3 + 2] = nz * inv;
  if (areas) areas[f] = 0.5f * len;
}

// ------------------------------------------------------------------ INT8 quantisation
// Element i belongs to channel (i / inner) % channels; scale / zero_point have `channels` entries (1 = per tensor).
__global__ void quantize_i8_kernel(const float* __restrict__ x, signed char* __restrict__ q,
                                   const float* __restrict__ scale, const float* __restrict__ zp, long long n,
                                   long long inner, int channels, int qmin, int qmax) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const int c = channels == 1 ? 0 : (int)((i / inner) % channels);
    const float v = rintf(x[i] / scale[c]) + zp[c];
    q[i] = (signed char)fminf(fmaxf(v, (float)qmin), (float)qmax);
  }
}
__global__ void dequantize_i8_kernel(const signed char* __restrict__ q, float* __restrict__ x,
                                     const float* __restrict__ scale, const float* __restrict__ zp, long long n,
                                     long long inner, int channels) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const int c = channels == 1 ? 0 : (int)((i / inner) % channels);
    x[i] = ((float)q[i] - zp[c]) * scale[c];
  }
}
__global__ void fake_quant_kernel(const float* __restrict__ x, float* __restrict__ y, const float* __restrict__ scale,
                                  const float* __restrict__ zp, long long n, long long inner, int channels, int qmin,
                                  int qmax) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const int c = channels == 1 ? 0 : (int)((i / inner) % channels);
    const float v = fminf(fmaxf(rintf(x[i] / scale[c]) + zp[c], (float)qmin), (float)qmax);
    y[i] = (v - zp[c]) * scale[c];
  }
}

// ------------------------------------------------------------------ Conv2d + BatchNorm + ReLU (inference)
// x [N,Cin,H,W], w [Cout,Cin,KH,KW], optional conv bias; BN folded on the fly: y = relu((conv + b - mean) * g/sqrt(var+eps) + beta).
// One thread per output element; the filter of the block's output channel is staged in shared memory.
__global__ void conv_bn_relu_kernel(const float* __restrict__ x, const float* __restrict__ w,
                                    const float* __restrict__ bias, const float* __restrict__ gamma,
                                    const float* __restrict__ beta, const float* __restrict__ mean,
                                    const float* __restrict__ var, float* __restrict__ y, int N, int Cin, int H, int W,
                                    int Cout, int KH, int KW, int stride, int pad, int OH, int OW, float eps,
                                    int relu) {
  extern __shared__ float sw[];
  const int co = blockIdx.y, n = blockIdx.z;
  const int fsz = Cin * KH * KW;
  for (int i = threadIdx.x; i < fsz; i += blockDim.x) sw[i] = w[(long long)co * fsz + i];
  __syncthreads();
  const int o = blockIdx.x * blockDim.x + threadIdx.x;
  if (o >= OH * OW) return;
  const int oh = o / OW, ow = o % OW;
  float acc = bias ? bias[co] : 0.f;
  const float* xn = x + (long long)n * Cin * H * W;
  for (int ci = 0; ci < Cin; ++ci)
    for (int kh = 0; kh < KH; ++kh) {
      const int ih = oh * stride - pad + kh;
      if (ih < 0 || ih >= H) continue;
      for (int kw = 0; kw < KW; ++kw) {
        const int iw = ow * stride - pad + kw;
        if (iw < 0 || iw >= W) continue;
        acc += xn[((long long)ci * H + ih) * W + iw] * sw[(ci * KH + kh) * KW + kw];
      }
    }
  if (gamma) acc = (acc - mean[co]) * rsqrtf(var[co] + eps) * gamma[co] + beta[co];
  if (relu) acc = fmaxf(acc, 0.f);
  y[(((long long)n * Cout + co) * OH + oh) * OW + ow] = acc;
}

// ------------------------------------------------------------------ BatchNorm (NCHW or NC with HW = 1)
// One block per channel: mean / biased variance over N*HW, running-stat update, then normalise.
__global__ void batchnorm_train_kernel(const float* __restrict__ x, float* __restrict__ y,
                                       const float* __restrict__ gamma, const float* __restrict__ beta,
                                       float* __restrict__ running_mean, float* __restrict__ running_var,
                                       float* __restrict__ save_mean, float* __restrict__ save_rstd, int N, int C,
                                       int HW, float eps, float momentum) {
  __shared__ float r1[32], r2[32];
  const int c = blockIdx.x;
  const long long cnt = (long long)N * HW;
  float s = 0.f, ss = 0.f;
  for (long long i = threadIdx.x; i < cnt; i += blockDim.x) {
    const float v = x[((i / HW) * C + c) * HW + (i % HW)];
    s += v;
    ss += v * v;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    s += __shfl_xor_sync(0xffffffffu, s, o);
    ss += __shfl_xor_sync(0xffffffffu, ss, o);
  }
  if ((threadIdx.x & 31) == 0) { r1[threadIdx.x >> 5] = s; r2[threadIdx.x >> 5] = ss; }
  __syncthreads();
  s = 0.f; ss = 0.f;
  for (int wv = 0; wv < (blockDim.x >> 5); ++wv) { s += r1[wv]; ss += r2[wv]; }
  const float mean = s / (float)cnt;
  const float var = fmaxf(ss / (float)cnt - mean * mean, 0.f);
  const float rstd = rsqrtf(var + eps);
  if (threadIdx.x == 0) {
    if (save_mean) save_mean[c] = mean;
    if (save_rstd) save_rstd[c] = rstd;
    if (running_mean) {
      const float unbiased = cnt > 1 ? var * (float)cnt / (float)(cnt - 1) : var;
      running_mean[c] = (1.f - momentum) * running_mean[c] + momentum * mean;
      running_var[c] = (1.f - momentum) * running_var[c] + momentum * unbiased;
    }
  }
  const float g = gamma ? gamma[c] : 1.f, b = beta ? beta[c] : 0.f;
  for (long long i = threadIdx.x; i < cnt; i += blockDim.x) {
    const long long off = ((i / HW) * C + c) * HW + (i % HW);
    y[off] = (x[off] - mean) * rstd * g + b;
  }
}

static inline int grid_for(long long n, int threads) {
  long long g = (n + threads - 1) / threads;
  const long long cap = (long long)sm_count() * 16;
  return (int)(g < 1 ? 1 : (g < cap ? g : cap));
}

}  // namespace gf

using namespace gf;
#define GF_RET() return cudaGetLastError() == cudaSuccess ? GFH_OK : GFH_CUDA

GF_API int gf_posenc(const float* x, float* out, long long n, int d, int num_freqs, int include_input, void* stream) {
  gf::enter();
  posenc_kernel<<<grid_for(n * d, 256), 256, 0, (cudaStream_t)stream>>>(x, out, n, d, num_freqs, include_input);
  GF_RET();
}
GF_API int gf_volume_render(const float* rgb, const float* sigma, const float* z, const float* ray_norm, float* color,
                            float* depth, float* acc, float* weights, int R, int S, int white_bg, void* stream) {
  gf::enter();
  if (R <= 0 || S <= 0) return GFH_BAD_ARG;
  volume_render_kernel<<<(R + 127) / 128, 128, 0, (cudaStream_t)stream>>>(rgb, sigma, z, ray_norm, color, depth, acc,
                                                                         weights, R, S, white_bg);
  GF_RET();
}
GF_API int gf_fps(const float* pts, int* idx, float* dist_scratch, int B, int N, int M, int start, void* stream) {
  gf::enter();
  if (B <= 0 || N <= 0 || M <= 0 || M > N) return GFH_BAD_ARG;
  fps_kernel<<<B, 512, 0, (cudaStream_t)stream>>>(pts, idx, dist_scratch, N, M, start);
  GF_RET();
}
GF_API int gf_knn(const float* pts, const float* queries, int* out, int B, int N, int Q, int K, void* stream) {
  gf::enter();
  if (K < 1 || K > 64 || K > N) return GFH_BAD_ARG;
  const long long total = (long long)B * Q;
  knn_kernel<<<(unsigned)((total + 127) / 128), 128, 0, (cudaStream_t)stream>>>(pts, queries, out, B, N, Q, K);
  GF_RET();
}
GF_API int gf_face_normals(const float* verts, const int* faces, float* normals, float* areas, int F, void* stream) {
  gf::enter();
  face_normals_kernel<<<(F + 255) / 256, 256, 0, (cudaStream_t)stream>>>(verts, faces, normals, areas, F);
  GF_RET();
}
GF_API int gf_quantize_i8(const float* x, void* q, const float* scale, const float* zp, long long n, long long inner,
                          int channels, int qmin, int qmax, void* stream) {
  gf::enter();
  quantize_i8_kernel<<<grid_for(n, 256), 256, 0, (cudaStream_t)stream>>>(x, (signed char*)q, scale, zp, n, inner,
                                                                        channels, qmin, qmax);
  GF_RET();
}
GF_API int gf_dequantize_i8(const void* q, float* x, const float* scale, const float* zp, long long n, long long inner,
                            int channels, void* stream) {
  gf::enter();
  dequantize_i8_kernel<<<grid_for(n, 256), 256, 0, (cudaStream_t)stream>>>((const signed char*)q, x, scale, zp, n,
                                                                          inner, channels);
  GF_RET();
}
GF_API int gf_fake_quant(const float* x, float* y, const float* scale, const float* zp, long long n, long long inner,
                         int channels, int qmin, int qmax, void* stream) {
  gf::enter();
  fake_quant_kernel<<<grid_for(n, 256), 256, 0, (cudaStream_t)stream>>>(x, y, scale, zp, n, inner, channels, qmin,
                                                                       qmax);
  GF_RET();
}
GF_API int gf_conv_bn_relu(const float* x, const float* w, const float* bias, const float* gamma, const float* beta,
                           const float* mean, const float* var, float* y, int N, int Cin, int H, int W, int Cout,
                           int KH, int KW, int stride, int pad, float eps, int relu, void* stream) {
  gf::enter();
  const int OH = (H + 2 * pad - KH) / stride + 1, OW = (W + 2 * pad - KW) / stride + 1;
  if (OH <= 0 || OW <= 0) return GFH_BAD_ARG;
  const size_t smem = (size_t)Cin * KH * KW * sizeof(float);
  if (smem > 160 * 1024) return GFH_TOO_LARGE;
  static gf::DeviceMax configured;
  if (smem > 48 * 1024 && smem > configured.get()) {
    if (cudaFuncSetAttribute(conv_bn_relu_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
      return GFH_CUDA;
    configured.set(smem);
  }
  dim3 grid((OH * OW + 127) / 128, Cout, N);
  conv_bn_relu_kernel<<<grid, 128, smem, (cudaStream_t)stream>>>(x, w, bias, gamma, beta, mean, var, y, N, Cin, H, W,
                                                                Cout, KH, KW, stride, pad, OH, OW, eps, relu);
  GF_RET();
}
GF_API int gf_batchnorm_train(const float* x, float* y, const float* gamma, const float* beta, float* running_mean,
                              float* running_var, float* save_mean, float* save_rstd, int N, int C, int HW, float eps,
                              float momentum, void* stream) {
  gf::enter();
  batchnorm_train_kernel<<<C, 256, 0, (cudaStream_t)stream>>>(x, y, gamma, beta, running_mean, running_var, save_mean,
                                                             save_rstd, N, C, HW, eps, momentum);
  GF_RET();
}


// ------------------------------------------------------------------ im2col for the tensor-core convolution
// x [N, C, H, W] fp32 -> cols [N * OH * OW, Kp] bf16 with column index (c * KH + ky) * KW + kx (the order of a
// weight viewed as [Cout, C * KH * KW]); columns >= C * KH * KW (padding to a multiple of 8) are zero.
namespace gf {
__global__ void im2col_bf16_kernel(const float* __restrict__ x, __nv_bfloat16* __restrict__ cols, int N, int C, int H,
                                   int W, int KH, int KW, int OH, int OW, int stride, int pad, int Kp) {
  const long long total = (long long)N * OH * OW * Kp;
  const int K = C * KH * KW;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int k = (int)(i % Kp);
    const long long row = i / Kp;
    float v = 0.f;
    if (k < K) {
      const int kx = k % KW, ky = (k / KW) % KH, c = k / (KW * KH);
      const int ox = (int)(row % OW), oy = (int)((row / OW) % OH), n = (int)(row / ((long long)OW * OH));
      const int iy = oy * stride - pad + ky, ix = ox * stride - pad + kx;
      if (iy >= 0 && iy < H && ix >= 0 && ix < W) v = x[(((long long)n * C + c) * H + iy) * W + ix];
    }
    cols[i] = __float2bfloat16(v);
  }
}
}  // namespace gf

// Channels-last variant for the bf16 inference path: x [N, H, W, C] bf16 with C a multiple of 8 ->
// cols [N * OH * OW, KH * KW * C] bf16 with column index (ky * KW + kx) * C + c (the order of a weight stored
// [Cout, KH, KW, C]). One thread moves one 16-byte group of 8 channels, so both sides are full-width accesses;
// taps that fall into the padding are written as zeros.
namespace gf {
// Block = 32 x 8 threads: threadIdx.y picks one of 8 output pixels, whose (n, oy, ox) is decomposed once; the 32
// threads of that pixel walk its KH * KW * C / 8 groups of 16 bytes, so a warp writes 512 contiguous bytes per step.
// c8_shift >= 0 when C / 8 is a power of two (the usual case): tap and channel group then come from a shift and a mask.
__global__ void __launch_bounds__(256)
im2col_nhwc_bf16_kernel(const uint4* __restrict__ x, uint4* __restrict__ cols, int N, int C8, int H, int W, int KH,
                        int KW, int OH, int OW, int stride, int pad, int c8_shift) {
  const int per_row = KH * KW * C8;
  const long long rows = (long long)N * OH * OW;
  for (long long row = (long long)blockIdx.x * 8 + threadIdx.y; row < rows; row += (long long)gridDim.x * 8) {
    const int ox = (int)(row % OW);
    const long long t = row / OW;
    const int oy = (int)(t % OH), n = (int)(t / OH);
    const int iy0 = oy * stride - pad, ix0 = ox * stride - pad;
    const uint4* xin = x + (long long)n * H * W * C8;
    uint4* out = cols + row * per_row;
    for (int j = threadIdx.x; j < per_row; j += 32) {
      int tap, c8;
      if (c8_shift >= 0) {
        tap = j >> c8_shift;
        c8 = j & (C8 - 1);
      } else {
        tap = j / C8;
        c8 = j - tap * C8;
      }
      const int ky = tap / KW, kx = tap - ky * KW;
      const int iy = iy0 + ky, ix = ix0 + kx;
      uint4 v = make_uint4(0u, 0u, 0u, 0u);
      if (iy >= 0 && iy < H && ix >= 0 && ix < W) v = xin[((long long)iy * W + ix) * C8 + c8];
      out[j] = v;
    }
  }
}
}  // namespace gf

GF_API int gf_im2col_nhwc_bf16(const void* x, void* cols, int N, int C, int H, int W, int KH, int KW, int stride,
                               int pad, void* stream) {
  gf::enter();
  if (C <= 0 || C % 8 || stride <= 0 || ((uintptr_t)x & 15) || ((uintptr_t)cols & 15)) return gf::GFH_BAD_ARG;
  const int OH = (H + 2 * pad - KH) / stride + 1, OW = (W + 2 * pad - KW) / stride + 1;
  if (OH <= 0 || OW <= 0) return gf::GFH_BAD_ARG;
  const long long rows = (long long)N * OH * OW;
  long long blocks = (rows + 7) / 8;
  const long long cap = (long long)gf::sm_count() * 16;
  if (blocks > cap) blocks = cap;
  const int C8 = C / 8;
  int shift = -1;
  if ((C8 & (C8 - 1)) == 0) {
    shift = 0;
    while ((1 << shift) < C8) ++shift;
  }
  gf::im2col_nhwc_bf16_kernel<<<(unsigned)blocks, dim3(32, 8), 0, (cudaStream_t)stream>>>(
      (const uint4*)x, (uint4*)cols, N, C8, H, W, KH, KW, OH, OW, stride, pad, shift);
  return cudaGetLastError() == cudaSuccess ? gf::GFH_OK : gf::GFH_CUDA;
}

// x [N, H, W, C] bf16 -> xp [N, H + pad, W + pad, C] with the image in the top-left corner and zeros in the `pad`
// trailing columns of every row and the `pad` trailing rows of every image (the layout the implicit convolution
// reads: one strip of zeros serves as right border of a row and left border of the next).
namespace gf {
// One block per padded image row: its first W * C8 groups of 16 bytes are a straight copy of the source row (when
// the row is inside the image), everything else is zero, so no thread divides anything.
__global__ void __launch_bounds__(256)
pad_nhwc_bf16_kernel(const uint4* __restrict__ x, uint4* __restrict__ xp, int N, int C8, int H, int W, int pad) {
  const int Hp = H + pad, Wp = W + pad;
  const int valid = W * C8, width = Wp * C8;
  for (int r = blockIdx.x; r < N * Hp; r += gridDim.x) {
    const int n = r / Hp, yy = r - n * Hp;
    const bool inside = yy < H;
    const uint4* src = x + ((long long)n * H + yy) * valid;
    uint4* dst = xp + (long long)r * width;
    for (int k = threadIdx.x; k < width; k += blockDim.x)
      dst[k] = (inside && k < valid) ? src[k] : make_uint4(0u, 0u, 0u, 0u);
  }
}
}  // namespace gf

GF_API int gf_pad_nhwc_bf16(const void* x, void* xp, int N, int C, int H, int W, int pad, void* stream) {
  gf::enter();
  if (C <= 0 || C % 8 || pad < 0 || N <= 0 || H <= 0 || W <= 0 || ((uintptr_t)x & 15) || ((uintptr_t)xp & 15))
    return gf::GFH_BAD_ARG;
  long long blocks = (long long)N * (H + pad);
  if (blocks > 0x7fffffffLL) return gf::GFH_BAD_ARG;
  const long long cap = (long long)gf::sm_count() * 32;
  if (blocks > cap) blocks = cap;
  gf::pad_nhwc_bf16_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>((const uint4*)x, (uint4*)xp, N, C / 8, H,
                                                                             W, pad);
  return cudaGetLastError() == cudaSuccess ? gf::GFH_OK : gf::GFH_CUDA;
}

GF_API int gf_im2col_bf16(const float* x, void* cols, int N, int C, int H, int W, int KH, int KW, int stride, int pad,
                          int Kp, void* stream) {
  gf::enter();
  const int OH = (H + 2 * pad - KH) / stride + 1, OW = (W + 2 * pad - KW) / stride + 1;
  if (OH <= 0 || OW <= 0 || Kp < C * KH * KW || Kp % 8) return gf::GFH_BAD_ARG;
  const long long total = (long long)N * OH * OW * Kp;
  long long blocks = (total + 255) / 256;
  const long long cap = (long long)gf::sm_count() * 16;
  if (blocks > cap) blocks = cap;
  gf::im2col_bf16_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(x, (__nv_bfloat16*)cols, N, C, H, W, KH, KW,
                                                                            OH, OW, stride, pad, Kp);
  return cudaGetLastError() == cudaSuccess ? gf::GFH_OK : gf::GFH_CUDA;
}
