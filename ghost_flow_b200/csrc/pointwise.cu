// Bandwidth-bound pointwise kernels: RoPE (both pairings, forward and backward, in place
// on a strided Q/K view), SwiGLU and GELU forward/backward, the small elementwise set
// (add, mul, relu, sigmoid, op-chain), row softmax and sum/max reductions.
//
// Math follows the reference's CPU code: RoPE interleaved pairs (ghostflow-nn/src/llama.rs:201-256)
// and half-split pairs (ghostflow-nn/src/transformer.rs:363-438); SwiGLU down(silu(gate)*up)
// (ghostflow-nn/src/llama.rs:266-286); tanh-form GELU (ghostflow-core/src/ops/activation.rs:101-112);
// op-code chain {0 ReLU, 1 GELU, 2 Sigmoid, 3 Tanh} (ghostflow-cuda/src/optimized_kernels.cu:254-286),
// here with the op list passed by value instead of re-read from global memory per element.
#include "gf_host.h"
#include "gf_ptx.cuh"

namespace gf {

__device__ __forceinline__ float gelu_tanh(float x) {
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;
  return 0.5f * x * (1.f + tanhf(k0 * (x + k1 * x * x * x)));
}
__device__ __forceinline__ float gelu_tanh_grad(float x) {
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;
  const float u = k0 * (x + k1 * x * x * x);
  const float t = tanhf(u);
  const float du = k0 * (1.f + 3.f * k1 * x * x);
  return 0.5f * (1.f + t) + 0.5f * x * (1.f - t * t) * du;
}
__device__ __forceinline__ float sigmoidf_(float x) { return 1.f / (1.f + __expf(-x)); }

// ------------------------------------------------------------------ RoPE
// x viewed as [T, H, D] with strides (row_stride, head_stride, 1) in elements. cos/sin tables are
// fp32 [S, D/2]; token t uses position (t % S) + pos_offset. sign = +1 forward, -1 backward.
// mode 0: half-split pairs (i, i + D/2); mode 1: interleaved pairs (2i, 2i+1).
__global__ void rope_kernel(__nv_bfloat16* __restrict__ x, const float* __restrict__ cos_t,
                            const float* __restrict__ sin_t, int T, int H, int D, long long row_stride,
                            long long head_stride, int S, int pos_offset, int mode, float sign) {
  const int half = D >> 1;
  const int pairs_per_vec = 8;  // 8 pairs per thread: two 16-byte loads (half-split) or two adjacent (interleaved)
  const int vecs_per_head = half / pairs_per_vec;
  const long long total = (long long)T * H * vecs_per_head;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const int v = (int)(idx % vecs_per_head);
    const long long th = idx / vecs_per_head;
    const int h = (int)(th % H);
    const long long t = th / H;
    const int pos = (int)(t % S) + pos_offset;
    __nv_bfloat16* base = x + t * row_stride + (long long)h * head_stride;
    const float* cp = cos_t + (long long)pos * half + v * pairs_per_vec;
    const float* sp = sin_t + (long long)pos * half + v * pairs_per_vec;
    float c[8], s[8];
    *reinterpret_cast<float4*>(c) = *reinterpret_cast<const float4*>(cp);
    *reinterpret_cast<float4*>(c + 4) = *reinterpret_cast<const float4*>(cp + 4);
    *reinterpret_cast<float4*>(s) = *reinterpret_cast<const float4*>(sp);
    *reinterpret_cast<float4*>(s + 4) = *reinterpret_cast<const float4*>(sp + 4);
    if (mode == 0) {
      uint4 ua = *reinterpret_cast<uint4*>(base + v * 8);
      uint4 ub = *reinterpret_cast<uint4*>(base + half + v * 8);
      uint32_t* pa = reinterpret_cast<uint32_t*>(&ua);
      uint32_t* pb = reinterpret_cast<uint32_t*>(&ub);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        float2 a = unpack_bf16x2(pa[q]), b = unpack_bf16x2(pb[q]);
        const float s0 = sign * s[2 * q], s1 = sign * s[2 * q + 1];
        float2 oa, ob;
        oa.x = a.x * c[2 * q] - b.x * s0;
        ob.x = b.x * c[2 * q] + a.x * s0;
        oa.y = a.y * c[2 * q + 1] - b.y * s1;
        ob.y = b.y * c[2 * q + 1] + a.y * s1;
        pa[q] = pack_bf16x2(oa.x, oa.y);
        pb[q] = pack_bf16x2(ob.x, ob.y);
      }
      *reinterpret_cast<uint4*>(base + v * 8) = ua;
      *reinterpret_cast<uint4*>(base + half + v * 8) = ub;
    } else {
      uint4 u0 = *reinterpret_cast<uint4*>(base + v * 16);
      uint4 u1 = *reinterpret_cast<uint4*>(base + v * 16 + 8);
      uint32_t* p0 = reinterpret_cast<uint32_t*>(&u0);
      uint32_t* p1 = reinterpret_cast<uint32_t*>(&u1);
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        uint32_t* pp = (q < 4) ? &p0[q] : &p1[q - 4];
        float2 a = unpack_bf16x2(*pp);
        const float sn = sign * s[q];
        *pp = pack_bf16x2(a.x * c[q] - a.y * sn, a.y * c[q] + a.x * sn);
      }
      *reinterpret_cast<uint4*>(base + v * 16) = u0;
      *reinterpret_cast<uint4*>(base + v * 16 + 8) = u1;
    }
  }
}

// ------------------------------------------------------------------ SwiGLU
// gu is [T, 2F] (gate columns [0,F), up columns [F,2F)); y = silu(g) * u is [T, F].
__global__ void swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ y, long long T,
                                  int F) {
  const int vpr = F >> 3;
  const long long total = T * vpr;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long t = idx / vpr;
    const int v = (int)(idx % vpr);
    const __nv_bfloat16* g = gu + t * 2 * F + v * 8;
    uint4 ug = *reinterpret_cast<const uint4*>(g);
    uint4 uu = *reinterpret_cast<const uint4*>(g + F);
    const uint32_t* pg = reinterpret_cast<const uint32_t*>(&ug);
    const uint32_t* pu = reinterpret_cast<const uint32_t*>(&uu);
    uint4 o;
    uint32_t* po = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      float2 a = unpack_bf16x2(pg[q]), b = unpack_bf16x2(pu[q]);
      po[q] = pack_bf16x2(a.x * sigmoidf_(a.x) * b.x, a.y * sigmoidf_(a.y) * b.y);
    }
    *reinterpret_cast<uint4*>(y + t * F + v * 8) = o;
  }
}
// dgu[T,2F]: dg = dy * u * (sig + g*sig*(1-sig)) ; du = dy * g * sig
__global__ void swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ gu, const __nv_bfloat16* __restrict__ dy,
                                  __nv_bfloat16* __restrict__ dgu, long long T, int F) {
  const int vpr = F >> 3;
  const long long total = T * vpr;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long t = idx / vpr;
    const int v = (int)(idx % vpr);
    const __nv_bfloat16* g = gu + t * 2 * F + v * 8;
    uint4 ug = *reinterpret_cast<const uint4*>(g);
    uint4 uu = *reinterpret_cast<const uint4*>(g + F);
    uint4 ud = *reinterpret_cast<const uint4*>(dy + t * F + v * 8);
    const uint32_t* pg = reinterpret_cast<const uint32_t*>(&ug);
    const uint32_t* pu = reinterpret_cast<const uint32_t*>(&uu);
    const uint32_t* pd = reinterpret_cast<const uint32_t*>(&ud);
    uint4 og, ou;
    uint32_t* pog = reinterpret_cast<uint32_t*>(&og);
    uint32_t* pou = reinterpret_cast<uint32_t*>(&ou);
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      float2 a = unpack_bf16x2(pg[q]), b = unpack_bf16x2(pu[q]), d = unpack_bf16x2(pd[q]);
      const float s0 = sigmoidf_(a.x), s1 = sigmoidf_(a.y);
      pog[q] = pack_bf16x2(d.x * b.x * (s0 + a.x * s0 * (1.f - s0)), d.y * b.y * (s1 + a.y * s1 * (1.f - s1)));
      pou[q] = pack_bf16x2(d.x * a.x * s0, d.y * a.y * s1);
    }
    *reinterpret_cast<uint4*>(dgu + t * 2 * F + v * 8) = og;
    *reinterpret_cast<uint4*>(dgu + t * 2 * F + F + v * 8) = ou;
  }
}

// ------------------------------------------------------------------ unary / binary elementwise (bf16 or fp32)
enum Op : int { OP_RELU = 0, OP_GELU = 1, OP_SIGMOID = 2, OP_TANH = 3, OP_SILU = 4 };
__device__ __forceinline__ float apply_op(int op, float x) {
  switch (op) {
    case OP_RELU: return fmaxf(x, 0.f);
    case OP_GELU: return gelu_tanh(x);
    case OP_SIGMOID: return sigmoidf_(x);
    case OP_TANH: return tanhf(x);
    default: return x * sigmoidf_(x);
  }
}
__device__ __forceinline__ float apply_op_grad(int op, float x) {
  switch (op) {
    case OP_RELU: return x > 0.f ? 1.f : 0.f;
    case OP_GELU: return gelu_tanh_grad(x);
    case OP_SIGMOID: { const float s = sigmoidf_(x); return s * (1.f - s); }
    case OP_TANH: { const float t = tanhf(x); return 1.f - t * t; }
    default: { const float s = sigmoidf_(x); return s + x * s * (1.f - s); }
  }
}
struct OpChain {
  int n;
  int ops[8];
};

template <typename T>
__device__ __forceinline__ float ldf(const T* p, long long i);
template <>
__device__ __forceinline__ float ldf<float>(const float* p, long long i) { return p[i]; }
template <>
__device__ __forceinline__ float ldf<__nv_bfloat16>(const __nv_bfloat16* p, long long i) {
  return __bfloat162float(p[i]);
}
template <typename T>
__device__ __forceinline__ void stf(T* p, long long i, float v);
template <>
__device__ __forceinline__ void stf<float>(float* p, long long i, float v) { p[i] = v; }
template <>
__device__ __forceinline__ void stf<__nv_bfloat16>(__nv_bfloat16* p, long long i, float v) {
  p[i] = __float2bfloat16(v);
}

// Generic chain kernel, 8 elements per thread iteration when aligned.
template <typename T>
__global__ void chain_fwd_kernel(const T* __restrict__ x, T* __restrict__ y, long long n, OpChain chain) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    float v = ldf(x, i);
    for (int k = 0; k < chain.n; ++k) v = apply_op(chain.ops[k], v);
    stf(y, i, v);
  }
}
__global__ void unary_fwd_bf16x8_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y,
                                        long long nvec, int op) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec;
       i += (long long)gridDim.x * blockDim.x) {
    uint4 u = reinterpret_cast<const uint4*>(x)[i];
    uint32_t* p = reinterpret_cast<uint32_t*>(&u);
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      float2 a = unpack_bf16x2(p[q]);
      p[q] = pack_bf16x2(apply_op(op, a.x), apply_op(op, a.y));
    }
    reinterpret_cast<uint4*>(y)[i] = u;
  }
}
// dx = dy * f'(x)
__global__ void unary_bwd_bf16x8_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ dy,
                                        __nv_bfloat16* __restrict__ dx, long long nvec, int op) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec;
       i += (long long)gridDim.x * blockDim.x) {
    uint4 u = reinterpret_cast<const uint4*>(x)[i];
    uint4 d = reinterpret_cast<const uint4*>(dy)[i];
    uint32_t* p = reinterpret_cast<uint32_t*>(&u);
    uint32_t* pd = reinterpret_cast<uint32_t*>(&d);
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      float2 a = unpack_bf16x2(p[q]), g = unpack_bf16x2(pd[q]);
      p[q] = pack_bf16x2(g.x * apply_op_grad(op, a.x), g.y * apply_op_grad(op, a.y));
    }
    reinterpret_cast<uint4*>(dx)[i] = u;
  }
}
template <typename T>
__global__ void binary_kernel(const T* __restrict__ a, const T* __restrict__ b, T* __restrict__ y, long long n,
                              int op /*0 add,1 mul,2 sub*/, float alpha) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const float av = ldf(a, i), bv = ldf(b, i);
    stf(y, i, op == 0 ? av + alpha * bv : (op == 1 ? av * bv : av - alpha * bv));
  }
}
// fp32 operands, four elements (16 bytes) per thread iteration.
__global__ void binary_f32x4_kernel(const float4* __restrict__ a, const float4* __restrict__ b, float4* __restrict__ y,
                                    long long nvec, int op, float alpha) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec;
       i += (long long)gridDim.x * blockDim.x) {
    const float4 u = a[i], v = b[i];
    float4 r;
    if (op == 0) {
      r = make_float4(u.x + alpha * v.x, u.y + alpha * v.y, u.z + alpha * v.z, u.w + alpha * v.w);
    } else if (op == 1) {
      r = make_float4(u.x * v.x, u.y * v.y, u.z * v.z, u.w * v.w);
    } else {
      r = make_float4(u.x - alpha * v.x, u.y - alpha * v.y, u.z - alpha * v.z, u.w - alpha * v.w);
    }
    y[i] = r;
  }
}
__global__ void chain_fwd_f32x4_kernel(const float4* __restrict__ x, float4* __restrict__ y, long long nvec,
                                       OpChain chain) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec;
       i += (long long)gridDim.x * blockDim.x) {
    float4 v = x[i];
    for (int k = 0; k < chain.n; ++k) {
      const int op = chain.ops[k];
      v = make_float4(apply_op(op, v.x), apply_op(op, v.y), apply_op(op, v.z), apply_op(op, v.w));
    }
    y[i] = v;
  }
}
__global__ void add_bf16x8_kernel(const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ b,
                                  __nv_bfloat16* __restrict__ y, long long nvec) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec;
       i += (long long)gridDim.x * blockDim.x) {
    uint4 ua = reinterpret_cast<const uint4*>(a)[i];
    uint4 ub = reinterpret_cast<const uint4*>(b)[i];
    uint32_t* pa = reinterpret_cast<uint32_t*>(&ua);
    uint32_t* pb = reinterpret_cast<uint32_t*>(&ub);
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      float2 x = unpack_bf16x2(pa[q]), z = unpack_bf16x2(pb[q]);
      pa[q] = pack_bf16x2(x.x + z.x, x.y + z.y);
    }
    reinterpret_cast<uint4*>(y)[i] = ua;
  }
}

// ------------------------------------------------------------------ reductions (fp32 result)
// mode 0 sum, 1 max. Two-stage: per-block partials then a single block folds them.
template <typename T>
__global__ void reduce_stage1_kernel(const T* __restrict__ x, float* __restrict__ partial, long long n, int mode) {
  __shared__ float red[32];
  float acc = mode == 0 ? 0.f : -INFINITY;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const float v = ldf(x, i);
    acc = mode == 0 ? acc + v : fmaxf(acc, v);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float t = __shfl_xor_sync(0xffffffffu, acc, o);
    acc = mode == 0 ? acc + t : fmaxf(acc, t);
  }
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : (mode == 0 ? 0.f : -INFINITY);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float u = __shfl_xor_sync(0xffffffffu, t, o);
      t = mode == 0 ? t + u : fmaxf(t, u);
    }
    if (threadIdx.x == 0) partial[blockIdx.x] = t;
  }
}
// fp32 input, four elements per load (n a multiple of 4, 16-byte aligned).
__global__ void reduce_stage1_f32x4_kernel(const float4* __restrict__ x, float* __restrict__ partial, long long nvec,
                                           int mode) {
  __shared__ float red[32];
  float acc = mode == 0 ? 0.f : -INFINITY;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec;
       i += (long long)gridDim.x * blockDim.x) {
    const float4 v = x[i];
    acc = mode == 0 ? acc + ((v.x + v.y) + (v.z + v.w)) : fmaxf(acc, fmaxf(fmaxf(v.x, v.y), fmaxf(v.z, v.w)));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float t = __shfl_xor_sync(0xffffffffu, acc, o);
    acc = mode == 0 ? acc + t : fmaxf(acc, t);
  }
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : (mode == 0 ? 0.f : -INFINITY);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float u = __shfl_xor_sync(0xffffffffu, t, o);
      t = mode == 0 ? t + u : fmaxf(t, u);
    }
    if (threadIdx.x == 0) partial[blockIdx.x] = t;
  }
}
__global__ void reduce_stage2_kernel(const float* __restrict__ partial, float* __restrict__ out, int nparts,
                                     int mode) {
  __shared__ float red[32];
  float acc = mode == 0 ? 0.f : -INFINITY;
  for (int i = threadIdx.x; i < nparts; i += blockDim.x) acc = mode == 0 ? acc + partial[i] : fmaxf(acc, partial[i]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float t = __shfl_xor_sync(0xffffffffu, acc, o);
    acc = mode == 0 ? acc + t : fmaxf(acc, t);
  }
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = red[0];
    for (int w = 1; w < (blockDim.x >> 5); ++w) t = mode == 0 ? t + red[w] : fmaxf(t, red[w]);
    out[0] = t;
  }
}

// ------------------------------------------------------------------ row softmax (last dim), any row length
template <typename T>
__global__ void softmax_rows_kernel(const T* __restrict__ x, T* __restrict__ y, int rows, int cols, int log_mode) {
  __shared__ float red[32];
  for (int r = blockIdx.x; r < rows; r += gridDim.x) {
    const T* xr = x + (long long)r * cols;
    float m = -INFINITY;
    for (int c = threadIdx.x; c < cols; c += blockDim.x) m = fmaxf(m, ldf(xr, c));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = m;
    __syncthreads();
    m = red[0];
    for (int w = 1; w < (blockDim.x >> 5); ++w) m = fmaxf(m, red[w]);
    float s = 0.f;
    for (int c = threadIdx.x; c < cols; c += blockDim.x) s += __expf(ldf(xr, c) - m);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
    __syncthreads();
    s = 0.f;
    for (int w = 0; w < (blockDim.x >> 5); ++w) s += red[w];
    const float inv = 1.f / s, ls = logf(s);
    T* yr = y + (long long)r * cols;
    for (int c = threadIdx.x; c < cols; c += blockDim.x) {
      const float v = ldf(xr, c) - m;
      stf(yr, c, log_mode ? v - ls : __expf(v) * inv);
    }
  }
}

// Rows of at most 256 * PER elements: the row stays in registers between the three steps (max, sum, write), so
// memory is read once and written once.
template <typename T, int PER>
__global__ void __launch_bounds__(256)
softmax_rows_reg_kernel(const T* __restrict__ x, T* __restrict__ y, int rows, int cols, int log_mode) {
  __shared__ float red[32];
  const int nw = blockDim.x >> 5;
  for (int r = blockIdx.x; r < rows; r += gridDim.x) {
    const T* xr = x + (long long)r * cols;
    float v[PER];
    float m = -INFINITY;
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      const int c = threadIdx.x + j * 256;
      v[j] = c < cols ? ldf(xr, c) : -INFINITY;
      m = fmaxf(m, v[j]);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = m;
    __syncthreads();
    m = red[0];
    for (int w = 1; w < nw; ++w) m = fmaxf(m, red[w]);
    float s = 0.f;
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      v[j] -= m;                                  // -inf for the columns past the end: exp gives 0
      s += __expf(v[j]);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
    __syncthreads();
    s = 0.f;
    for (int w = 0; w < nw; ++w) s += red[w];
    const float inv = 1.f / s, ls = logf(s);
    T* yr = y + (long long)r * cols;
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      const int c = threadIdx.x + j * 256;
      if (c < cols) stf(yr, c, log_mode ? v[j] - ls : __expf(v[j]) * inv);
    }
  }
}

static inline int ew_grid(long long n, int threads) {
  long long g = (n + threads - 1) / threads;
  const long long cap = (long long)sm_count() * 16;
  return (int)(g < cap ? (g > 0 ? g : 1) : cap);
}

// x *= *scalar unless *scalar == 1 (the usual case for the gradient of a loss that is the root of the backward
// pass): the decision is taken on the device, so the host never has to read the scalar.
__global__ void scale_by_dev_scalar_kernel(__nv_bfloat16* __restrict__ x, long long n, const float* __restrict__ scalar) {
  const float s = *scalar;
  if (s == 1.f) return;
  const long long nvec = n >> 3;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec;
       i += (long long)gridDim.x * blockDim.x) {
    uint4 u = reinterpret_cast<uint4*>(x)[i];
    uint32_t* w = reinterpret_cast<uint32_t*>(&u);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      __nv_bfloat162 v = *reinterpret_cast<__nv_bfloat162*>(&w[j]);
      float2 f = __bfloat1622float2(v);
      v = __floats2bfloat162_rn(f.x * s, f.y * s);
      w[j] = *reinterpret_cast<uint32_t*>(&v);
    }
    reinterpret_cast<uint4*>(x)[i] = u;
  }
  if (blockIdx.x == 0 && threadIdx.x == 0)
    for (long long i = nvec << 3; i < n; ++i) x[i] = __float2bfloat16(__bfloat162float(x[i]) * s);
}

}  // namespace gf

using namespace gf;
#define GF_RET() return cudaGetLastError() == cudaSuccess ? GFH_OK : GFH_CUDA

GF_API int gf_rope(void* x, const float* cos_t, const float* sin_t, int T, int H, int D, long long row_stride,
                   long long head_stride, int S, int pos_offset, int mode, int backward, void* stream) {
  gf::enter();
  if (D % 16 || (row_stride % 8) || (head_stride % 8) || T <= 0) return GFH_BAD_ARG;
  const long long total = (long long)T * H * (D / 16);
  rope_kernel<<<ew_grid(total, 256), 256, 0, (cudaStream_t)stream>>>((__nv_bfloat16*)x, cos_t, sin_t, T, H, D,
                                                                    row_stride, head_stride, S, pos_offset, mode,
                                                                    backward ? -1.f : 1.f);
  GF_RET();
}
// x: bf16 [n], 16-byte aligned; scalar: one fp32 on the device.
GF_API int gf_scale_by_dev_scalar(void* x, long long n, const float* scalar, void* stream) {
  gf::enter();
  if (!x || !scalar || n <= 0 || (reinterpret_cast<uintptr_t>(x) & 15)) return GFH_BAD_ARG;
  scale_by_dev_scalar_kernel<<<ew_grid(n / 8 + 1, 256), 256, 0, (cudaStream_t)stream>>>((__nv_bfloat16*)x, n, scalar);
  GF_RET();
}
GF_API int gf_swiglu_fwd(const void* gu, void* y, long long T, int F, void* stream) {
  gf::enter();
  if (F % 8) return GFH_BAD_ARG;
  swiglu_fwd_kernel<<<ew_grid(T * (F / 8), 256), 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)gu,
                                                                                (__nv_bfloat16*)y, T, F);
  GF_RET();
}
GF_API int gf_swiglu_bwd(const void* gu, const void* dy, void* dgu, long long T, int F, void* stream) {
  gf::enter();
  if (F % 8) return GFH_BAD_ARG;
  swiglu_bwd_kernel<<<ew_grid(T * (F / 8), 256), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)gu, (const __nv_bfloat16*)dy, (__nv_bfloat16*)dgu, T, F);
  GF_RET();
}
// dtype: 0 = fp32, 1 = bf16
GF_API int gf_unary_fwd(const void* x, void* y, long long n, int op, int dtype, void* stream) {
  gf::enter();
  if (dtype == 1 && n % 8 == 0 && ((uintptr_t)x % 16 == 0) && ((uintptr_t)y % 16 == 0)) {
    unary_fwd_bf16x8_kernel<<<ew_grid(n / 8, 256), 256, 0, (cudaStream_t)stream>>>(
        (const __nv_bfloat16*)x, (__nv_bfloat16*)y, n / 8, op);
  } else {
    OpChain c;
    c.n = 1;
    c.ops[0] = op;
    if (dtype == 1)
      chain_fwd_kernel<__nv_bfloat16><<<ew_grid(n, 256), 256, 0, (cudaStream_t)stream>>>(
          (const __nv_bfloat16*)x, (__nv_bfloat16*)y, n, c);
    else if (n % 4 == 0 && ((uintptr_t)x % 16 == 0) && ((uintptr_t)y % 16 == 0))
      chain_fwd_f32x4_kernel<<<ew_grid(n / 4, 256), 256, 0, (cudaStream_t)stream>>>((const float4*)x, (float4*)y,
                                                                                  n / 4, c);
    else
      chain_fwd_kernel<float><<<ew_grid(n, 256), 256, 0, (cudaStream_t)stream>>>((const float*)x, (float*)y, n, c);
  }
  GF_RET();
}
GF_API int gf_unary_bwd_bf16(const void* x, const void* dy, void* dx, long long n, int op, void* stream) {
  gf::enter();
  if (n % 8) return GFH_BAD_ARG;
  unary_bwd_bf16x8_kernel<<<ew_grid(n / 8, 256), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)x, (const __nv_bfloat16*)dy, (__nv_bfloat16*)dx, n / 8, op);
  GF_RET();
}
GF_API int gf_op_chain(const void* x, void* y, long long n, const int* ops, int nops, int dtype, void* stream) {
  gf::enter();
  if (nops < 0 || nops > 8) return GFH_BAD_ARG;
  OpChain c;
  c.n = nops;
  for (int i = 0; i < nops; ++i) c.ops[i] = ops[i];
  if (dtype == 1)
    chain_fwd_kernel<__nv_bfloat16><<<ew_grid(n, 256), 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)x,
                                                                                      (__nv_bfloat16*)y, n, c);
  else if (n % 4 == 0 && ((uintptr_t)x % 16 == 0) && ((uintptr_t)y % 16 == 0))
    chain_fwd_f32x4_kernel<<<ew_grid(n / 4, 256), 256, 0, (cudaStream_t)stream>>>((const float4*)x, (float4*)y, n / 4,
                                                                                c);
  else
    chain_fwd_kernel<float><<<ew_grid(n, 256), 256, 0, (cudaStream_t)stream>>>((const float*)x, (float*)y, n, c);
  GF_RET();
}
GF_API int gf_binary(const void* a, const void* b, void* y, long long n, int op, float alpha, int dtype,
                     void* stream) {
  gf::enter();
  if (dtype == 1 && op == 0 && alpha == 1.f && n % 8 == 0 && ((uintptr_t)a % 16 == 0) && ((uintptr_t)b % 16 == 0) &&
      ((uintptr_t)y % 16 == 0)) {
    add_bf16x8_kernel<<<ew_grid(n / 8, 256), 256, 0, (cudaStream_t)stream>>>(
        (const __nv_bfloat16*)a, (const __nv_bfloat16*)b, (__nv_bfloat16*)y, n / 8);
  } else if (dtype == 1) {
    binary_kernel<__nv_bfloat16><<<ew_grid(n, 256), 256, 0, (cudaStream_t)stream>>>(
        (const __nv_bfloat16*)a, (const __nv_bfloat16*)b, (__nv_bfloat16*)y, n, op, alpha);
  } else if (n % 4 == 0 && ((uintptr_t)a % 16 == 0) && ((uintptr_t)b % 16 == 0) && ((uintptr_t)y % 16 == 0)) {
    binary_f32x4_kernel<<<ew_grid(n / 4, 256), 256, 0, (cudaStream_t)stream>>>((const float4*)a, (const float4*)b,
                                                                             (float4*)y, n / 4, op, alpha);
  } else {
    binary_kernel<float><<<ew_grid(n, 256), 256, 0, (cudaStream_t)stream>>>((const float*)a, (const float*)b,
                                                                           (float*)y, n, op, alpha);
  }
  GF_RET();
}
// partial: fp32 scratch of at least 1024 floats; out: fp32 scalar.
GF_API int gf_reduce(const void* x, float* partial, float* out, long long n, int mode, int dtype, void* stream) {
  gf::enter();
  int g = ew_grid(n, 256);
  if (g > 1024) g = 1024;
  if (dtype == 1)
    reduce_stage1_kernel<__nv_bfloat16><<<g, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)x, partial, n,
                                                                            mode);
  else if (n % 4 == 0 && ((uintptr_t)x % 16 == 0)) {
    g = ew_grid(n / 4, 256);
    if (g > 1024) g = 1024;
    reduce_stage1_f32x4_kernel<<<g, 256, 0, (cudaStream_t)stream>>>((const float4*)x, partial, n / 4, mode);
  } else
    reduce_stage1_kernel<float><<<g, 256, 0, (cudaStream_t)stream>>>((const float*)x, partial, n, mode);
  reduce_stage2_kernel<<<1, 256, 0, (cudaStream_t)stream>>>(partial, out, g, mode);
  gf::note_extra_launches(1);
  GF_RET();
}
GF_API int gf_softmax_rows(const void* x, void* y, int rows, int cols, int log_mode, int dtype, void* stream) {
  gf::enter();
  int g = rows < sm_count() * 8 ? rows : sm_count() * 8;
  cudaStream_t st = (cudaStream_t)stream;
#define GF_SOFTMAX_REG(T_, PER_)                                                                              \
  softmax_rows_reg_kernel<T_, PER_><<<g, 256, 0, st>>>((const T_*)x, (T_*)y, rows, cols, log_mode)
  if (dtype == 1) {
    if (cols <= 256 * 4) GF_SOFTMAX_REG(__nv_bfloat16, 4);
    else if (cols <= 256 * 16) GF_SOFTMAX_REG(__nv_bfloat16, 16);
    else if (cols <= 256 * 32) GF_SOFTMAX_REG(__nv_bfloat16, 32);
    else softmax_rows_kernel<__nv_bfloat16><<<g, 256, 0, st>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)y, rows, cols,
                                                              log_mode);
  } else {
    if (cols <= 256 * 4) GF_SOFTMAX_REG(float, 4);
    else if (cols <= 256 * 16) GF_SOFTMAX_REG(float, 16);
    else if (cols <= 256 * 32) GF_SOFTMAX_REG(float, 32);
    else softmax_rows_kernel<float><<<g, 256, 0, st>>>((const float*)x, (float*)y, rows, cols, log_mode);
  }
#undef GF_SOFTMAX_REG
  GF_RET();
}

// ------------------------------------------------------------------ fp32 -> (hi, lo) bf16 split for 3-term GEMMs
// x = hi + lo + O(2^-16 |x|) with hi = bf16(x), lo = bf16(x - hi). An fp32 product A B is then approximated to
// about 2^-16 relative by hi_A hi_B + hi_A lo_B + lo_A hi_B, which is ONE bf16 GEMM over a three times longer
// contraction: A' = [hi_A | hi_A | lo_A] (columns), B' = [hi_B ; lo_B ; hi_B] (rows). This kernel writes x's three
// copies into such a buffer: copy j of element (r, c) lands at out[r * out_pitch + c + off[j]], and copy
// `lo_slot` (1 or 2) is the low part.
namespace gf {
__global__ void split_bf16_cat_kernel(const float* __restrict__ x, __nv_bfloat16* __restrict__ out, long long rows,
                                      int cols, long long in_pitch, long long out_pitch, long long off1, long long off2,
                                      int lo_slot) {
  const long long total = rows * cols;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / cols;
    const int c = (int)(i - r * cols);
    const float v = x[r * in_pitch + c];
    const __nv_bfloat16 hi = __float2bfloat16(v);
    const __nv_bfloat16 lo = __float2bfloat16(v - __bfloat162float(hi));
    __nv_bfloat16* o = out + r * out_pitch + c;
    o[0] = hi;
    o[off1] = lo_slot == 1 ? lo : hi;
    o[off2] = lo_slot == 2 ? lo : hi;
  }
}
// Same, eight columns per thread: two 16-byte loads, three 16-byte stores (cols, pitches and offsets multiples of 8,
// 16-byte aligned pointers).
__global__ void split_bf16_cat_x8_kernel(const float* __restrict__ x, __nv_bfloat16* __restrict__ out, long long rows,
                                         int cols8, long long in_pitch, long long out_pitch, long long off1,
                                         long long off2, int lo_slot) {
  const long long total = rows * cols8;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / cols8;
    const int c = (int)(i - r * cols8) * 8;
    const float4 a = *reinterpret_cast<const float4*>(x + r * in_pitch + c);
    const float4 b = *reinterpret_cast<const float4*>(x + r * in_pitch + c + 4);
    const float v[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
    uint32_t hi[4], lo[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const __nv_bfloat16 h0 = __float2bfloat16(v[2 * q]), h1 = __float2bfloat16(v[2 * q + 1]);
      hi[q] = pack_bf16x2(__bfloat162float(h0), __bfloat162float(h1));
      lo[q] = pack_bf16x2(v[2 * q] - __bfloat162float(h0), v[2 * q + 1] - __bfloat162float(h1));
    }
    const uint4 H = make_uint4(hi[0], hi[1], hi[2], hi[3]), L = make_uint4(lo[0], lo[1], lo[2], lo[3]);
    __nv_bfloat16* o = out + r * out_pitch + c;
    *reinterpret_cast<uint4*>(o) = H;
    *reinterpret_cast<uint4*>(o + off1) = lo_slot == 1 ? L : H;
    *reinterpret_cast<uint4*>(o + off2) = lo_slot == 2 ? L : H;
  }
}
}  // namespace gf

GF_API int gf_split_bf16_cat(const float* x, void* out, long long rows, int cols, long long in_pitch,
                             long long out_pitch, long long off1, long long off2, int lo_slot, void* stream) {
  gf::enter();
  if (rows <= 0 || cols <= 0 || (lo_slot != 1 && lo_slot != 2)) return GFH_BAD_ARG;
  if (cols % 8 == 0 && in_pitch % 4 == 0 && out_pitch % 8 == 0 && off1 % 8 == 0 && off2 % 8 == 0 &&
      ((uintptr_t)x & 15) == 0 && ((uintptr_t)out & 15) == 0) {
    split_bf16_cat_x8_kernel<<<ew_grid(rows * (cols / 8), 256), 256, 0, (cudaStream_t)stream>>>(
        x, (__nv_bfloat16*)out, rows, cols / 8, in_pitch, out_pitch, off1, off2, lo_slot);
  } else {
    split_bf16_cat_kernel<<<ew_grid(rows * cols, 256), 256, 0, (cudaStream_t)stream>>>(
        x, (__nv_bfloat16*)out, rows, cols, in_pitch, out_pitch, off1, off2, lo_slot);
  }
  GF_RET();
}
