// libghostflow.so: GhostFlow's C ABI (include/ghostflow.h) over a small host tensor.
// Counterpart of ghostflow-ffi/src/lib.rs:60-337; add/mul follow NumPy broadcasting
// (ghostflow-core/src/shape.rs:50-82), matmul is cache-blocked and multi-threaded.
#include <algorithm>
#include <cstring>
#include <new>
#include <string>
#include <thread>
#include <vector>

#include "include/ghostflow.h"

#define GF_EXPORT extern "C" __attribute__((visibility("default")))

struct GhostFlowTensor {
  std::vector<uintptr_t> shape;
  std::vector<float> data;
};

namespace {
thread_local std::string g_last_error;

GhostFlowError fail(GhostFlowError e, const char* msg) {
  g_last_error = msg;
  return e;
}

size_t numel(const std::vector<uintptr_t>& s) {
  size_t n = 1;
  for (auto d : s) n *= d;
  return n;
}

GhostFlowError make(const uintptr_t* shape, uintptr_t nd, float fill, GhostFlowTensor** out) {
  if (!out || (!shape && nd)) return fail(NullPointer, "null pointer argument");
  try {
    auto* t = new GhostFlowTensor();
    t->shape.assign(shape, shape + nd);
    t->data.assign(numel(t->shape), fill);
    *out = t;
  } catch (const std::bad_alloc&) {
    return fail(AllocationFailed, "out of memory");
  }
  return Success;
}

bool broadcast_shape(const std::vector<uintptr_t>& a, const std::vector<uintptr_t>& b, std::vector<uintptr_t>& o) {
  const size_t nd = std::max(a.size(), b.size());
  o.assign(nd, 1);
  for (size_t i = 0; i < nd; ++i) {
    const uintptr_t da = i < nd - a.size() ? 1 : a[i - (nd - a.size())];
    const uintptr_t db = i < nd - b.size() ? 1 : b[i - (nd - b.size())];
    if (da != db && da != 1 && db != 1) return false;
    o[i] = std::max(da, db);
  }
  return true;
}

template <typename F>
GhostFlowError binary(const GhostFlowTensor* a, const GhostFlowTensor* b, GhostFlowTensor** out, F f) {
  if (!a || !b || !out) return fail(NullPointer, "null pointer argument");
  std::vector<uintptr_t> os;
  if (!broadcast_shape(a->shape, b->shape, os)) return fail(InvalidShape, "shapes cannot be broadcast together");
  GhostFlowError e = make(os.data(), os.size(), 0.f, out);
  if (e != Success) return e;
  GhostFlowTensor* o = *out;
  const size_t nd = os.size(), n = o->data.size();
  if (a->shape == b->shape) {
    for (size_t i = 0; i < n; ++i) o->data[i] = f(a->data[i], b->data[i]);
    return Success;
  }
  // strides with 0 on broadcast dimensions
  std::vector<size_t> sa(nd, 0), sb(nd, 0);
  auto strides = [&](const std::vector<uintptr_t>& s, std::vector<size_t>& st) {
    size_t acc = 1;
    for (size_t k = s.size(); k-- > 0;) {
      st[nd - s.size() + k] = s[k] == 1 ? 0 : acc;
      acc *= s[k];
    }
  };
  strides(a->shape, sa);
  strides(b->shape, sb);
  std::vector<size_t> idx(nd, 0);
  size_t ia = 0, ib = 0;
  for (size_t i = 0; i < n; ++i) {
    o->data[i] = f(a->data[ia], b->data[ib]);
    for (size_t k = nd; k-- > 0;) {
      ++idx[k];
      ia += sa[k];
      ib += sb[k];
      if (idx[k] < os[k]) break;
      ia -= sa[k] * idx[k];
      ib -= sb[k] * idx[k];
      idx[k] = 0;
    }
  }
  return Success;
}

void matmul_block(const float* A, const float* B, float* C, size_t m0, size_t m1, size_t K, size_t N) {
  constexpr size_t BK = 64, BN = 256;
  for (size_t k0 = 0; k0 < K; k0 += BK)
    for (size_t n0 = 0; n0 < N; n0 += BN) {
      const size_t k1 = std::min(K, k0 + BK), n1 = std::min(N, n0 + BN);
      for (size_t i = m0; i < m1; ++i)
        for (size_t k = k0; k < k1; ++k) {
          const float a = A[i * K + k];
          const float* brow = B + k * N;
          float* crow = C + i * N;
          for (size_t j = n0; j < n1; ++j) crow[j] += a * brow[j];
        }
    }
}
}  // namespace

GF_EXPORT GhostFlowError ghostflow_init(void) {
  g_last_error.clear();
  return Success;
}
GF_EXPORT const char* ghostflow_version(void) {
  static const char v[] = "ghost_flow_b200 0.1.0 (GhostFlow C ABI 1.2)";
  char* s = static_cast<char*>(malloc(sizeof(v)));
  if (s) memcpy(s, v, sizeof(v));
  return s;
}
GF_EXPORT void ghostflow_free_string(char* s) { free(s); }

GF_EXPORT GhostFlowError ghostflow_tensor_create(const float* data, uintptr_t data_len, const uintptr_t* shape,
                                                 uintptr_t shape_len, GhostFlowTensor** out) {
  if (!data || !shape || !out) return fail(NullPointer, "null pointer argument");
  std::vector<uintptr_t> s(shape, shape + shape_len);
  if (numel(s) != data_len) return fail(InvalidShape, "shape does not match the number of elements");
  GhostFlowError e = make(shape, shape_len, 0.f, out);
  if (e != Success) return e;
  memcpy((*out)->data.data(), data, data_len * sizeof(float));
  return Success;
}
GF_EXPORT GhostFlowError ghostflow_tensor_zeros(const uintptr_t* shape, uintptr_t n, GhostFlowTensor** out) {
  return make(shape, n, 0.f, out);
}
GF_EXPORT GhostFlowError ghostflow_tensor_ones(const uintptr_t* shape, uintptr_t n, GhostFlowTensor** out) {
  return make(shape, n, 1.f, out);
}
GF_EXPORT void ghostflow_tensor_free(GhostFlowTensor* t) { delete t; }

GF_EXPORT GhostFlowError ghostflow_tensor_shape(const GhostFlowTensor* t, uintptr_t* out_shape, uintptr_t* out_ndim) {
  if (!t || !out_ndim) return fail(NullPointer, "null pointer argument");
  *out_ndim = t->shape.size();
  if (out_shape) std::copy(t->shape.begin(), t->shape.end(), out_shape);
  return Success;
}
GF_EXPORT GhostFlowError ghostflow_tensor_data(const GhostFlowTensor* t, float* out_data, uintptr_t* out_len) {
  if (!t || !out_len) return fail(NullPointer, "null pointer argument");
  *out_len = t->data.size();
  if (out_data) memcpy(out_data, t->data.data(), t->data.size() * sizeof(float));
  return Success;
}
GF_EXPORT GhostFlowError ghostflow_tensor_add(const GhostFlowTensor* a, const GhostFlowTensor* b, GhostFlowTensor** out) {
  return binary(a, b, out, [](float x, float y) { return x + y; });
}
GF_EXPORT GhostFlowError ghostflow_tensor_mul(const GhostFlowTensor* a, const GhostFlowTensor* b, GhostFlowTensor** out) {
  return binary(a, b, out, [](float x, float y) { return x * y; });
}
GF_EXPORT GhostFlowError ghostflow_tensor_matmul(const GhostFlowTensor* a, const GhostFlowTensor* b, GhostFlowTensor** out) {
  if (!a || !b || !out) return fail(NullPointer, "null pointer argument");
  if (a->shape.size() < 2 || b->shape.size() < 2) return fail(InvalidShape, "matmul needs tensors of rank >= 2");
  const size_t M = a->shape[a->shape.size() - 2], K = a->shape.back();
  const size_t K2 = b->shape[b->shape.size() - 2], N = b->shape.back();
  if (K != K2) return fail(InvalidShape, "inner dimensions of matmul do not match");
  std::vector<uintptr_t> ba(a->shape.begin(), a->shape.end() - 2), bb(b->shape.begin(), b->shape.end() - 2), bo;
  if (!broadcast_shape(ba, bb, bo)) return fail(InvalidShape, "batch dimensions cannot be broadcast together");
  std::vector<uintptr_t> os = bo;
  os.push_back(M);
  os.push_back(N);
  GhostFlowError e = make(os.data(), os.size(), 0.f, out);
  if (e != Success) return e;
  const size_t nb = numel(bo), na = numel(ba), nbb = numel(bb);
  for (size_t bi = 0; bi < nb; ++bi) {
    const float* A = a->data.data() + (na == 1 ? 0 : (bi % na)) * M * K;
    const float* B = b->data.data() + (nbb == 1 ? 0 : (bi % nbb)) * K * N;
    float* C = (*out)->data.data() + bi * M * N;
    unsigned nt = std::max(1u, std::min<unsigned>(std::thread::hardware_concurrency(), 16));
    if (M * N * K < (1u << 22)) nt = 1;
    if (nt == 1) {
      matmul_block(A, B, C, 0, M, K, N);
    } else {
      std::vector<std::thread> th;
      const size_t per = (M + nt - 1) / nt;
      for (unsigned t = 0; t < nt; ++t) {
        const size_t m0 = t * per, m1 = std::min(M, m0 + per);
        if (m0 < m1) th.emplace_back(matmul_block, A, B, C, m0, m1, K, N);
      }
      for (auto& x : th) x.join();
    }
  }
  return Success;
}
GF_EXPORT GhostFlowError ghostflow_tensor_reshape(const GhostFlowTensor* t, const uintptr_t* new_shape,
                                                  uintptr_t n, GhostFlowTensor** out) {
  if (!t || !new_shape || !out) return fail(NullPointer, "null pointer argument");
  std::vector<uintptr_t> s(new_shape, new_shape + n);
  if (numel(s) != t->data.size()) return fail(InvalidShape, "reshape changes the number of elements");
  GhostFlowError e = make(new_shape, n, 0.f, out);
  if (e != Success) return e;
  (*out)->data = t->data;
  return Success;
}
GF_EXPORT const char* ghostflow_get_last_error(void) { return g_last_error.c_str(); }
