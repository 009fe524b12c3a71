"""ctypes binding of the C++ CPU oracle (``csrc/cpu_ref.cpp``): the reference's formulas as plain fp32 loops.

Every function takes and returns contiguous fp32 torch CPU tensors. The oracle is independent of PyTorch's own CPU
kernels, so agreement between the two (and with the GPU kernels) is a three-way check."""
from __future__ import annotations

import ctypes

import torch

from . import _lib

_BOUND = False


def _bind():
    global _BOUND
    lib = _lib.host_lib()
    if not _BOUND:
        P, I, L, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float
        sig = {"gfref_matmul": [P, P, P, I, I, I], "gfref_linear": [P, P, P, P, I, I, I], "gfref_gelu_tanh": [P, P, L],
               "gfref_gelu_fast_tanh": [P, P, L], "gfref_silu": [P, P, L], "gfref_softmax_rows": [P, P, I, I],
               "gfref_layernorm": [P, P, P, P, I, I, F], "gfref_rmsnorm": [P, P, P, I, I, F],
               "gfref_cross_entropy": [P, P, P, I, I], "gfref_adam_step": [P, P, P, P, L, F, F, F, F, F, I, I],
               "gfref_argmax_rows": [P, P, I, I], "gfref_attention": [P, P, P, P, I, I, I, F, I],
               "gfref_conv2d": [P, P, P, P, I, I, I, I, I, I, I, I, I]}
        for n, a in sig.items():
            getattr(lib, n).argtypes = a
            getattr(lib, n).restype = None
        lib.gfref_cross_entropy.restype = F
        _BOUND = True
    return lib


def _f(t):
    return t.detach().to(torch.float32).contiguous().cpu()


def _p(t):
    return t.data_ptr() if t is not None else None


def matmul(a, b):
    a, b = _f(a), _f(b)
    c = torch.empty(a.shape[0], b.shape[1])
    _bind().gfref_matmul(_p(a), _p(b), _p(c), a.shape[0], a.shape[1], b.shape[1])
    return c


def linear(x, w, bias=None):
    x, w = _f(x), _f(w)
    bias = _f(bias) if bias is not None else None
    y = torch.empty(x.shape[0], w.shape[0])
    _bind().gfref_linear(_p(x), _p(w), _p(bias), _p(y), x.shape[0], x.shape[1], w.shape[0])
    return y


def _unary(name, x):
    x = _f(x)
    y = torch.empty_like(x)
    getattr(_bind(), name)(_p(x), _p(y), x.numel())
    return y


def gelu(x, fast_tanh: bool = False):
    """Exact-tanh GELU; ``fast_tanh=True`` gives the reference's default-build rational approximation."""
    return _unary("gfref_gelu_fast_tanh" if fast_tanh else "gfref_gelu_tanh", x)


def silu(x):
    return _unary("gfref_silu", x)


def softmax(x):
    x = _f(x)
    y = torch.empty_like(x)
    _bind().gfref_softmax_rows(_p(x), _p(y), x.numel() // x.shape[-1], x.shape[-1])
    return y


def layer_norm(x, w=None, b=None, eps=1e-5):
    x = _f(x)
    w, b = (_f(w) if w is not None else None), (_f(b) if b is not None else None)
    y = torch.empty_like(x)
    _bind().gfref_layernorm(_p(x), _p(w), _p(b), _p(y), x.numel() // x.shape[-1], x.shape[-1], eps)
    return y


def rms_norm(x, w=None, eps=1e-6):
    x = _f(x)
    w = _f(w) if w is not None else None
    y = torch.empty_like(x)
    _bind().gfref_rmsnorm(_p(x), _p(w), _p(y), x.numel() // x.shape[-1], x.shape[-1], eps)
    return y


def cross_entropy(logits, targets, with_grad: bool = False):
    logits = _f(logits)
    t = targets.detach().to(torch.int64).contiguous().cpu()
    g = torch.empty_like(logits) if with_grad else None
    loss = _bind().gfref_cross_entropy(_p(logits), _p(t), _p(g), logits.shape[0], logits.shape[1])
    return (loss, g) if with_grad else loss


def adam_step(p, m, v, g, *, lr, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.0, step=1, decoupled=True):
    """In place on fp32 contiguous CPU tensors p, m, v."""
    g = _f(g)
    _bind().gfref_adam_step(_p(p), _p(m), _p(v), _p(g), p.numel(), lr, beta1, beta2, eps, weight_decay, step,
                            1 if decoupled else 0)


def argmax(x):
    x = _f(x)
    o = torch.empty(x.shape[0])
    _bind().gfref_argmax_rows(_p(x), _p(o), x.shape[0], x.shape[1])
    return o


def attention(q, k, v, causal=False, scale=None):
    """q, k, v: [heads, seq, dim]."""
    q, k, v = _f(q), _f(k), _f(v)
    o = torch.empty_like(q)
    h, s, d = q.shape
    _bind().gfref_attention(_p(q), _p(k), _p(v), _p(o), h, s, d, scale if scale is not None else d ** -0.5, 1 if causal else 0)
    return o


def conv2d(x, w, bias=None, stride=1, padding=0):
    x, w = _f(x), _f(w)
    bias = _f(bias) if bias is not None else None
    n, cin, h, wd = x.shape
    cout, _, kh, kw = w.shape
    y = torch.empty(n, cout, (h + 2 * padding - kh) // stride + 1, (wd + 2 * padding - kw) // stride + 1)
    _bind().gfref_conv2d(_p(x), _p(w), _p(bias), _p(y), n, cin, h, wd, cout, kh, kw, stride, padding)
    return y
