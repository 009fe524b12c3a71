"""Element-wise arithmetic, full reductions and row softmax for the tensor API on the library's own kernels.

``binary`` (add / sub / mul), ``unary_any`` (relu / gelu / sigmoid / tanh / silu for fp32 as well as bf16),
``reduce_all`` (sum / max) and ``softmax_rows`` launch ``gf_binary``, ``gf_unary_fwd``, ``gf_reduce`` and
``gf_softmax_rows`` when the operands are dense CUDA tensors of one dtype (fp32 or bf16) that carry no autograd
graph; everything else (broadcasting, integer types, tensors that require grad, CPU) is computed by PyTorch. These
are the kernels behind the reference's intended names ``ghostflow_add_f32 / mul / relu / gelu / sigmoid / sum /
max / softmax`` (ghostflow-cuda/src/kernels/mod.rs:47-110) and its CPU loops in
ghostflow-core/src/ops/arithmetic.rs:20-120, activation.rs:9-216 and reduction.rs:10-117.
"""
from __future__ import annotations

import torch

from . import _lib

_BIN = {"add": 0, "mul": 1, "sub": 2}
_UN = {"relu": 0, "gelu": 1, "sigmoid": 2, "tanh": 3, "silu": 4}
_DT = {torch.float32: 0, torch.bfloat16: 1}
_PARTIAL: dict = {}


def _plain(*ts) -> bool:
    first = ts[0]
    for t in ts:
        if not (torch.is_tensor(t) and t.is_cuda and t.dtype in _DT and t.dtype == first.dtype and t.is_contiguous()
                and t.numel() > 0 and not (torch.is_grad_enabled() and t.requires_grad)):
            return False
    return True


def binary(a, b, op: str, alpha: float = 1.0):
    """``a + alpha * b``, ``a - alpha * b`` or ``a * b``."""
    if torch.is_tensor(b) and _plain(a, b) and a.shape == b.shape:
        y = torch.empty_like(a)
        _lib.check_rc(_lib.cuda_lib().gf_binary(a.data_ptr(), b.data_ptr(), y.data_ptr(), a.numel(), _BIN[op],
                                                float(alpha), _DT[a.dtype], _lib.stream_ptr()), "gf_binary")
        return y
    if op == "mul":
        return torch.mul(a, b)
    return torch.add(a, b, alpha=alpha) if op == "add" else torch.sub(a, b, alpha=alpha)


def unary_any(x, name: str):
    if _plain(x):
        y = torch.empty_like(x)
        _lib.check_rc(_lib.cuda_lib().gf_unary_fwd(x.data_ptr(), y.data_ptr(), x.numel(), _UN[name], _DT[x.dtype],
                                                   _lib.stream_ptr()), "gf_unary_fwd")
        return y
    from .fused import unary

    return unary(x, name)


def reduce_all(x, mode: str = "sum"):
    """Sum or maximum over every element; the result is an fp32 scalar tensor on ``x``'s device."""
    if _plain(x):
        key = x.device.index
        part = _PARTIAL.get(key)
        if part is None:
            part = _PARTIAL[key] = torch.empty(4096, dtype=torch.float32, device=x.device)
        out = torch.empty((), dtype=torch.float32, device=x.device)
        _lib.check_rc(_lib.cuda_lib().gf_reduce(x.data_ptr(), part.data_ptr(), out.data_ptr(), x.numel(),
                                                0 if mode == "sum" else 1, _DT[x.dtype], _lib.stream_ptr()),
                      "gf_reduce")
        return out
    return (x.sum() if mode == "sum" else x.max()).float()


def softmax_rows(x, log: bool = False):
    """Softmax (or log-softmax) over the last dimension."""
    if _plain(x) and x.dim() >= 1:
        cols = x.shape[-1]
        y = torch.empty_like(x)
        _lib.check_rc(_lib.cuda_lib().gf_softmax_rows(x.data_ptr(), y.data_ptr(), x.numel() // cols, cols,
                                                      1 if log else 0, _DT[x.dtype], _lib.stream_ptr()),
                      "gf_softmax_rows")
        return y
    return torch.log_softmax(x, -1) if log else torch.softmax(x, -1)
