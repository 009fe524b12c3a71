// CPU oracle: the reference's formulas restated as plain C++ loops over fp32, behind a C ABI (host library).
// Used by tests as an independent check of the GPU kernels and of the PyTorch CPU paths, and by the timed CPU
// baseline of the tiny-GPT configuration.
//
// Formulas and where the reference states them:
//   GELU, exact-tanh form             ghostflow-core/src/ops/activation.rs:101-112
//   GELU with the rational tanh       ghostflow-core/src/ops/simd.rs:136-143 (default build; x(27+x^2)/(27+9x^2), clamp +-3)
//   softmax / log-softmax             ghostflow-core/src/ops/activation.rs
//   LayerNorm (biased variance)       ghostflow-nn/src/norm.rs:222-224,256-266
//   RMSNorm                           ghostflow-nn/src/llama.rs:154-185
//   cross entropy (mean over rows)    ghostflow-nn/src/loss.rs:89-102
//   Adam / AdamW                      ghostflow-optim/src/adam.rs:162-197
//   matmul (row-major, ikj order)     ghostflow-core/src/ops/matmul.rs:91-170
//   argmax returned as float          ghostflow-core/src/ops/reduction.rs:89-96
//   scaled-dot-product attention      ghostflow-nn/src/attention.rs:11-49
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <vector>

#define GFREF_API extern "C" __attribute__((visibility("default")))

GFREF_API void gfref_matmul(const float* a, const float* b, float* c, int m, int k, int n) {
  std::memset(c, 0, sizeof(float) * (size_t)m * n);
  for (int i = 0; i < m; ++i)
    for (int p = 0; p < k; ++p) {
      const float av = a[(size_t)i * k + p];
      const float* br = b + (size_t)p * n;
      float* cr = c + (size_t)i * n;
      for (int j = 0; j < n; ++j) cr[j] += av * br[j];
    }
}

// y[m, n] = x[m, k] w[n, k]^T + bias
GFREF_API void gfref_linear(const float* x, const float* w, const float* bias, float* y, int m, int k, int n) {
  for (int i = 0; i < m; ++i)
    for (int j = 0; j < n; ++j) {
      float s = bias ? bias[j] : 0.f;
      const float* xr = x + (size_t)i * k;
      const float* wr = w + (size_t)j * k;
      for (int p = 0; p < k; ++p) s += xr[p] * wr[p];
      y[(size_t)i * n + j] = s;
    }
}

GFREF_API void gfref_gelu_tanh(const float* x, float* y, long long n) {
  const float c = 0.7978845608028654f;
  for (long long i = 0; i < n; ++i) y[i] = 0.5f * x[i] * (1.f + std::tanh(c * (x[i] + 0.044715f * x[i] * x[i] * x[i])));
}

GFREF_API void gfref_gelu_fast_tanh(const float* x, float* y, long long n) {
  const float c = 0.7978845608028654f;
  for (long long i = 0; i < n; ++i) {
    float t = c * (x[i] + 0.044715f * x[i] * x[i] * x[i]);
    t = std::max(-3.f, std::min(3.f, t));
    const float th = t * (27.f + t * t) / (27.f + 9.f * t * t);
    y[i] = 0.5f * x[i] * (1.f + th);
  }
}

GFREF_API void gfref_silu(const float* x, float* y, long long n) {
  for (long long i = 0; i < n; ++i) y[i] = x[i] / (1.f + std::exp(-x[i]));
}

GFREF_API void gfref_softmax_rows(const float* x, float* y, int rows, int cols) {
  for (int r = 0; r < rows; ++r) {
    const float* xr = x + (size_t)r * cols;
    float* yr = y + (size_t)r * cols;
    float mx = xr[0];
    for (int j = 1; j < cols; ++j) mx = std::max(mx, xr[j]);
    float s = 0.f;
    for (int j = 0; j < cols; ++j) { yr[j] = std::exp(xr[j] - mx); s += yr[j]; }
    for (int j = 0; j < cols; ++j) yr[j] /= s;
  }
}

GFREF_API void gfref_layernorm(const float* x, const float* w, const float* b, float* y, int rows, int cols, float eps) {
  for (int r = 0; r < rows; ++r) {
    const float* xr = x + (size_t)r * cols;
    float mean = 0.f, var = 0.f;
    for (int j = 0; j < cols; ++j) mean += xr[j];
    mean /= cols;
    for (int j = 0; j < cols; ++j) var += (xr[j] - mean) * (xr[j] - mean);
    var /= cols;
    const float rstd = 1.f / std::sqrt(var + eps);
    for (int j = 0; j < cols; ++j)
      y[(size_t)r * cols + j] = (xr[j] - mean) * rstd * (w ? w[j] : 1.f) + (b ? b[j] : 0.f);
  }
}

GFREF_API void gfref_rmsnorm(const float* x, const float* w, float* y, int rows, int cols, float eps) {
  for (int r = 0; r < rows; ++r) {
    const float* xr = x + (size_t)r * cols;
    float ms = 0.f;
    for (int j = 0; j < cols; ++j) ms += xr[j] * xr[j];
    const float rstd = 1.f / std::sqrt(ms / cols + eps);
    for (int j = 0; j < cols; ++j) y[(size_t)r * cols + j] = xr[j] * rstd * (w ? w[j] : 1.f);
  }
}

// Mean over rows of -log softmax at the target; also writes d(loss)/d(logits) when grad != nullptr.
GFREF_API float gfref_cross_entropy(const float* logits, const long long* targets, float* grad, int rows, int cols) {
  double total = 0.0;
  for (int r = 0; r < rows; ++r) {
    const float* xr = logits + (size_t)r * cols;
    float mx = xr[0];
    for (int j = 1; j < cols; ++j) mx = std::max(mx, xr[j]);
    double s = 0.0;
    for (int j = 0; j < cols; ++j) s += std::exp((double)xr[j] - mx);
    const double lse = mx + std::log(s);
    total += lse - xr[targets[r]];
    if (grad)
      for (int j = 0; j < cols; ++j)
        grad[(size_t)r * cols + j] = (float)((std::exp((double)xr[j] - lse) - (j == targets[r] ? 1.0 : 0.0)) / rows);
  }
  return (float)(total / rows);
}

// One Adam step. decoupled != 0: AdamW (p -= lr * wd * p before the update); else L2 added to the gradient.
GFREF_API void gfref_adam_step(float* p, float* m, float* v, const float* g, long long n, float lr, float beta1,
                               float beta2, float eps, float weight_decay, int step, int decoupled) {
  const float bc1 = 1.f - std::pow(beta1, (float)step), bc2 = 1.f - std::pow(beta2, (float)step);
  for (long long i = 0; i < n; ++i) {
    float gi = g[i];
    if (!decoupled) gi += weight_decay * p[i];
    m[i] = beta1 * m[i] + (1.f - beta1) * gi;
    v[i] = beta2 * v[i] + (1.f - beta2) * gi * gi;
    if (decoupled) p[i] -= lr * weight_decay * p[i];
    p[i] -= lr * (m[i] / bc1) / (std::sqrt(v[i] / bc2) + eps);
  }
}

GFREF_API void gfref_argmax_rows(const float* x, float* out, int rows, int cols) {
  for (int r = 0; r < rows; ++r) {
    int best = 0;
    for (int j = 1; j < cols; ++j)
      if (x[(size_t)r * cols + j] > x[(size_t)r * cols + best]) best = j;
    out[r] = (float)best;
  }
}

// q [h, s, d], k/v [h, s, d] -> o [h, s, d]; optional causal mask.
GFREF_API void gfref_attention(const float* q, const float* k, const float* v, float* o, int heads, int s, int d,
                               float scale, int causal) {
  std::vector<float> row(s);
  for (int h = 0; h < heads; ++h)
    for (int i = 0; i < s; ++i) {
      const float* qi = q + ((size_t)h * s + i) * d;
      const int lim = causal ? i + 1 : s;
      float mx = -INFINITY;
      for (int j = 0; j < lim; ++j) {
        const float* kj = k + ((size_t)h * s + j) * d;
        float acc = 0.f;
        for (int p = 0; p < d; ++p) acc += qi[p] * kj[p];
        row[j] = acc * scale;
        mx = std::max(mx, row[j]);
      }
      float sum = 0.f;
      for (int j = 0; j < lim; ++j) { row[j] = std::exp(row[j] - mx); sum += row[j]; }
      float* oi = o + ((size_t)h * s + i) * d;
      for (int p = 0; p < d; ++p) oi[p] = 0.f;
      for (int j = 0; j < lim; ++j) {
        const float w = row[j] / sum;
        const float* vj = v + ((size_t)h * s + j) * d;
        for (int p = 0; p < d; ++p) oi[p] += w * vj[p];
      }
    }
}

// Direct NCHW convolution, weights [cout, cin, kh, kw].
GFREF_API void gfref_conv2d(const float* x, const float* w, const float* bias, float* y, int n, int cin, int h, int wd,
                            int cout, int kh, int kw, int stride, int pad) {
  const int ho = (h + 2 * pad - kh) / stride + 1, wo = (wd + 2 * pad - kw) / stride + 1;
  for (int b = 0; b < n; ++b)
    for (int co = 0; co < cout; ++co)
      for (int oy = 0; oy < ho; ++oy)
        for (int ox = 0; ox < wo; ++ox) {
          float acc = bias ? bias[co] : 0.f;
          for (int ci = 0; ci < cin; ++ci)
            for (int ky = 0; ky < kh; ++ky) {
              const int iy = oy * stride - pad + ky;
              if (iy < 0 || iy >= h) continue;
              for (int kx = 0; kx < kw; ++kx) {
                const int ix = ox * stride - pad + kx;
                if (ix < 0 || ix >= wd) continue;
                acc += x[(((size_t)b * cin + ci) * h + iy) * wd + ix] * w[(((size_t)co * cin + ci) * kh + ky) * kw + kx];
              }
            }
          y[(((size_t)b * cout + co) * ho + oy) * wo + ox] = acc;
        }
}
