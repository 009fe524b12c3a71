// Softmax cross-entropy (fused forward + gradient, logits read from HBM once) and the
// flat fused AdamW / Adam / SGD updates on fp32 master weights with a bf16 copy-out.
//
// Cross-entropy: mean over rows of -log_softmax(logits)[target]
// (ghostflow-nn/src/loss.rs:75-103; gradient softmax - onehot, ghostflow-autograd/src/backward.rs:171-191).
// AdamW: p*(1 - lr*wd) - lr * mhat / (sqrt(vhat) + eps), m and v from the raw gradient
// (ghostflow-optim/src/adam.rs:162-197); Adam with L2-coupled decay (adam.rs:52-95);
// SGD with momentum/dampening/nesterov (ghostflow-optim/src/sgd.rs:54-93).
#include "gf_host.h"
#include "gf_ptx.cuh"

namespace gf {

constexpr int XENT_THREADS = 512;

// One CTA per row. The row is staged in shared memory as bf16 while the max is found, so the
// logits are read from global memory exactly once; dlogits overwrite the logits in place
// (or go to a separate buffer). loss_rows[t] = logsumexp - x[target]; ignored rows give 0.
__global__ void __launch_bounds__(XENT_THREADS)
xent_fused_kernel(const __nv_bfloat16* __restrict__ logits, const long long* __restrict__ targets,
                  float* __restrict__ loss_rows, __nv_bfloat16* __restrict__ dlogits, int T, int V, long long ld,
                  float grad_scale, long long ignore_index) {
  extern __shared__ __align__(16) uint8_t xs_raw[];
  __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(xs_raw);
  __shared__ float red[32];
  // Rows move as 16-byte vectors. The host guarantees ld % 8 == 0 and ld >= round_up(V, 8), so the last vector of a
  // row whose V is not a multiple of 8 lies inside the row's pitch: its columns >= V are read as -inf (they add
  // nothing to the sum) and get gradient 0.
  const int nv = (V + 7) >> 3;
  for (int row = blockIdx.x; row < T; row += gridDim.x) {
    const __nv_bfloat16* xr = logits + (long long)row * ld;
    const long long tgt = targets[row];
    float m = -INFINITY;
    for (int v = threadIdx.x; v < nv; v += XENT_THREADS) {
      uint4 u = *reinterpret_cast<const uint4*>(xr + v * 8);
      if (v * 8 + 8 > V) {
        unsigned short* h = reinterpret_cast<unsigned short*>(&u);
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (v * 8 + j >= V) h[j] = 0xFF80;   // bf16 -inf
      }
      *reinterpret_cast<uint4*>(xs + v * 8) = u;
      const uint32_t* p = reinterpret_cast<const uint32_t*>(&u);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        float2 a = unpack_bf16x2(p[q]);
        m = fmaxf(m, fmaxf(a.x, a.y));
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = m;
    __syncthreads();
    m = red[0];
#pragma unroll
    for (int w = 1; w < XENT_THREADS / 32; ++w) m = fmaxf(m, red[w]);
    float s = 0.f;
    for (int v = threadIdx.x; v < nv; v += XENT_THREADS) {
      uint4 u = *reinterpret_cast<const uint4*>(xs + v * 8);
      const uint32_t* p = reinterpret_cast<const uint32_t*>(&u);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        float2 a = unpack_bf16x2(p[q]);
        s += __expf(a.x - m) + __expf(a.y - m);
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
    __syncthreads();
    s = 0.f;
#pragma unroll
    for (int w = 0; w < XENT_THREADS / 32; ++w) s += red[w];
    const bool ignored = (tgt == ignore_index) || tgt < 0 || tgt >= V;
    if (threadIdx.x == 0)
      loss_rows[row] = ignored ? 0.f : (logf(s) + m - __bfloat162float(xs[tgt]));
    if (dlogits) {
      const float inv = ignored ? 0.f : grad_scale / s;
      __nv_bfloat16* dr = dlogits + (long long)row * ld;
      for (int v = threadIdx.x; v < nv; v += XENT_THREADS) {
        uint4 u = *reinterpret_cast<const uint4*>(xs + v * 8);
        uint32_t* p = reinterpret_cast<uint32_t*>(&u);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          float2 a = unpack_bf16x2(p[q]);
          float g0 = __expf(a.x - m) * inv, g1 = __expf(a.y - m) * inv;
          const int c = v * 8 + q * 2;
          if (!ignored) {
            if (c == tgt) g0 -= grad_scale;
            if (c + 1 == tgt) g1 -= grad_scale;
          }
          p[q] = pack_bf16x2(g0, g1);
        }
        *reinterpret_cast<uint4*>(dr + v * 8) = u;
      }
    }
    __syncthreads();
  }
}

// ------------------------------------------------------------------ flat optimizers
struct AdamArgs {
  float lr, beta1, beta2, eps, wd, bc1, bc2, grad_scale;
  int decoupled;  // 1 = AdamW, 0 = Adam (L2 added to the gradient)
};

// grad is bf16 or fp32; p/m/v fp32; optional bf16 copy of the updated weights. `skip` (device int)
// non-zero turns the launch into a no-op (loss-scaler found inf/nan).
template <typename G>
__global__ void adam_flat_kernel(float* __restrict__ p, float* __restrict__ m, float* __restrict__ v,
                                 const G* __restrict__ g, __nv_bfloat16* __restrict__ p_lp, long long n, AdamArgs a,
                                 const int* __restrict__ skip, const int* __restrict__ step_dev) {
  if (skip && *skip) return;
  if (step_dev) {   // step number kept on the device (a launch recorded in a CUDA graph is replayed with frozen arguments)
    const float t = (float)*step_dev;
    a.bc1 = 1.f - powf(a.beta1, t);
    a.bc2 = 1.f - powf(a.beta2, t);
  }
  const long long nvec = n >> 2;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec;
       i += (long long)gridDim.x * blockDim.x) {
    float4 pv = reinterpret_cast<float4*>(p)[i];
    float4 mv = reinterpret_cast<float4*>(m)[i];
    float4 vv = reinterpret_cast<float4*>(v)[i];
    float gr[4];
    if (sizeof(G) == 4) {
      float4 gv = reinterpret_cast<const float4*>(g)[i];
      gr[0] = gv.x; gr[1] = gv.y; gr[2] = gv.z; gr[3] = gv.w;
    } else {
      uint2 gu = reinterpret_cast<const uint2*>(g)[i];
      float2 a0 = unpack_bf16x2(gu.x), a1 = unpack_bf16x2(gu.y);
      gr[0] = a0.x; gr[1] = a0.y; gr[2] = a1.x; gr[3] = a1.y;
    }
    float* pp = reinterpret_cast<float*>(&pv);
    float* mp = reinterpret_cast<float*>(&mv);
    float* vp = reinterpret_cast<float*>(&vv);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float gj = gr[j] * a.grad_scale;
      if (!a.decoupled) gj += a.wd * pp[j];
      mp[j] = a.beta1 * mp[j] + (1.f - a.beta1) * gj;
      vp[j] = a.beta2 * vp[j] + (1.f - a.beta2) * gj * gj;
      const float mh = mp[j] / a.bc1, vh = vp[j] / a.bc2;
      float pj = pp[j];
      if (a.decoupled) pj *= (1.f - a.lr * a.wd);
      pp[j] = pj - a.lr * mh / (sqrtf(vh) + a.eps);
    }
    reinterpret_cast<float4*>(p)[i] = pv;
    reinterpret_cast<float4*>(m)[i] = mv;
    reinterpret_cast<float4*>(v)[i] = vv;
    if (p_lp) {
      uint2 o;
      o.x = pack_bf16x2(pp[0], pp[1]);
      o.y = pack_bf16x2(pp[2], pp[3]);
      reinterpret_cast<uint2*>(p_lp)[i] = o;
    }
  }
  // tail (n % 4) handled by the first threads of block 0
  if (blockIdx.x == 0 && threadIdx.x < (n & 3)) {
    const long long i = (nvec << 2) + threadIdx.x;
    float gj = (sizeof(G) == 4 ? reinterpret_cast<const float*>(g)[i]
                               : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(g)[i])) *
               a.grad_scale;
    if (!a.decoupled) gj += a.wd * p[i];
    m[i] = a.beta1 * m[i] + (1.f - a.beta1) * gj;
    v[i] = a.beta2 * v[i] + (1.f - a.beta2) * gj * gj;
    float pj = p[i];
    if (a.decoupled) pj *= (1.f - a.lr * a.wd);
    pj -= a.lr * (m[i] / a.bc1) / (sqrtf(v[i] / a.bc2) + a.eps);
    p[i] = pj;
    if (p_lp) p_lp[i] = __float2bfloat16(pj);
  }
}

template <typename G>
__global__ void sgd_flat_kernel(float* __restrict__ p, float* __restrict__ buf, const G* __restrict__ g,
                                __nv_bfloat16* __restrict__ p_lp, long long n, float lr, float momentum,
                                float dampening, float wd, int nesterov, int first_step, float grad_scale) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    float gj = (sizeof(G) == 4 ? reinterpret_cast<const float*>(g)[i]
                               : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(g)[i])) *
               grad_scale;
    gj += wd * p[i];
    if (momentum != 0.f) {
      float b = first_step ? gj : momentum * buf[i] + (1.f - dampening) * gj;
      buf[i] = b;
      gj = nesterov ? gj + momentum * b : b;
    }
    const float pj = p[i] - lr * gj;
    p[i] = pj;
    if (p_lp) p_lp[i] = __float2bfloat16(pj);
  }
}

// Sum of squares of a flat gradient into out[0] (atomic), plus a non-finite flag into out[1].
template <typename G>
__global__ void sumsq_kernel(const G* __restrict__ g, long long n, float* __restrict__ out) {
  __shared__ float red[32];
  float acc = 0.f;
  int bad = 0;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const float v = sizeof(G) == 4 ? reinterpret_cast<const float*>(g)[i]
                                   : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(g)[i]);
    acc += v * v;
    bad |= !isfinite(v);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  bad = __any_sync(0xffffffffu, bad);
  if ((threadIdx.x & 31) == 0) {
    red[threadIdx.x >> 5] = acc;
    if (bad) out[1] = 1.f;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int w = 0; w < (blockDim.x >> 5); ++w) t += red[w];
    atomicAdd(out, t);
  }
}

static inline int flat_grid(long long n) {
  long long g = (n + 1023) / 1024;
  // four CTAs (1024 threads) per SM at most: these kernels are HBM-bound and usually run beside compute kernels of another
  // stream, which must still find free thread slots and registers on every SM
  const long long cap = (long long)sm_count() * 4;
  return (int)(g < cap ? (g > 0 ? g : 1) : cap);
}

}  // namespace gf

using namespace gf;

// dlogits may equal logits (in place) or be null (loss only). ld = row pitch in elements.
GF_API int gf_xent_fused(const void* logits, const long long* targets, float* loss_rows, void* dlogits, int T, int V,
                         long long ld, float grad_scale, long long ignore_index, void* stream) {
  gf::enter();
  const long long v8 = ((long long)V + 7) / 8 * 8;
  if (V <= 0 || ld % 8 || ld < v8 || T <= 0) return GFH_BAD_ARG;
  if ((reinterpret_cast<uintptr_t>(logits) & 15) || (reinterpret_cast<uintptr_t>(dlogits) & 15)) return GFH_BAD_ARG;
  const size_t smem = (size_t)v8 * 2;
  if (smem > 200 * 1024) return GFH_TOO_LARGE;
  static gf::DeviceMax configured;
  if (smem > configured.get()) {
    if (cudaFuncSetAttribute(xent_fused_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=
        cudaSuccess)
      return GFH_CUDA;
    configured.set(smem);
  }
  xent_fused_kernel<<<T, XENT_THREADS, smem, (cudaStream_t)stream>>>((const __nv_bfloat16*)logits, targets,
                                                                    loss_rows, (__nv_bfloat16*)dlogits, T, V, ld,
                                                                    grad_scale, ignore_index);
  return cudaGetLastError() == cudaSuccess ? GFH_OK : GFH_CUDA;
}

// grad_dtype: 0 fp32, 1 bf16. p_lp may be null. skip may be null.
// step_dev (may be null): device int holding the step number; when given, `step` is ignored.
GF_API int gf_adam_flat_dev(float* p, float* m, float* v, const void* g, void* p_lp, long long n, float lr, float beta1,
                            float beta2, float eps, float wd, int step, float grad_scale, int decoupled,
                            int grad_dtype, const int* skip, const int* step_dev, void* stream) {
  gf::enter();
  if (n <= 0) return GFH_OK;
  static gf::DeviceOnce configured;
  if (configured.todo()) {
    prefer_max_smem(adam_flat_kernel<__nv_bfloat16>);
    prefer_max_smem(adam_flat_kernel<float>);
    configured.mark();
  }
  AdamArgs a;
  a.lr = lr; a.beta1 = beta1; a.beta2 = beta2; a.eps = eps; a.wd = wd; a.grad_scale = grad_scale;
  a.bc1 = 1.f - powf(beta1, (float)step);
  a.bc2 = 1.f - powf(beta2, (float)step);
  a.decoupled = decoupled;
  if (grad_dtype == 1)
    adam_flat_kernel<__nv_bfloat16><<<flat_grid(n), 256, 0, (cudaStream_t)stream>>>(
        p, m, v, (const __nv_bfloat16*)g, (__nv_bfloat16*)p_lp, n, a, skip, step_dev);
  else
    adam_flat_kernel<float><<<flat_grid(n), 256, 0, (cudaStream_t)stream>>>(
        p, m, v, (const float*)g, (__nv_bfloat16*)p_lp, n, a, skip, step_dev);
  return cudaGetLastError() == cudaSuccess ? GFH_OK : GFH_CUDA;
}

GF_API int gf_adam_flat(float* p, float* m, float* v, const void* g, void* p_lp, long long n, float lr, float beta1,
                        float beta2, float eps, float wd, int step, float grad_scale, int decoupled, int grad_dtype,
                        const int* skip, void* stream) {
  return gf_adam_flat_dev(p, m, v, g, p_lp, n, lr, beta1, beta2, eps, wd, step, grad_scale, decoupled, grad_dtype,
                          skip, nullptr, stream);
}

GF_API int gf_sgd_flat(float* p, float* buf, const void* g, void* p_lp, long long n, float lr, float momentum,
                       float dampening, float wd, int nesterov, int first_step, float grad_scale, int grad_dtype,
                       void* stream) {
  gf::enter();
  if (n <= 0) return GFH_OK;
  if (grad_dtype == 1)
    sgd_flat_kernel<__nv_bfloat16><<<flat_grid(n), 256, 0, (cudaStream_t)stream>>>(
        p, buf, (const __nv_bfloat16*)g, (__nv_bfloat16*)p_lp, n, lr, momentum, dampening, wd, nesterov, first_step,
        grad_scale);
  else
    sgd_flat_kernel<float><<<flat_grid(n), 256, 0, (cudaStream_t)stream>>>(
        p, buf, (const float*)g, (__nv_bfloat16*)p_lp, n, lr, momentum, dampening, wd, nesterov, first_step,
        grad_scale);
  return cudaGetLastError() == cudaSuccess ? GFH_OK : GFH_CUDA;
}

// out: fp32[2] = {sum of squares (accumulated), non-finite flag}; caller zeroes it first.
GF_API int gf_grad_sumsq(const void* g, long long n, float* out, int grad_dtype, void* stream) {
  gf::enter();
  if (n <= 0) return GFH_OK;
  if (grad_dtype == 1)
    sumsq_kernel<__nv_bfloat16><<<flat_grid(n), 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)g, n, out);
  else
    sumsq_kernel<float><<<flat_grid(n), 256, 0, (cudaStream_t)stream>>>((const float*)g, n, out);
  return cudaGetLastError() == cudaSuccess ? GFH_OK : GFH_CUDA;
}
