"""Flat (multi-tensor-free) optimizer kernels: one launch updates a whole contiguous shard.

``adam_flat`` covers Adam (L2-coupled decay) and AdamW (decoupled), ``sgd_flat`` covers SGD with
momentum / dampening / Nesterov; both write the bf16 working copy of the weights in the same pass.
Formulas: ghostflow-optim/src/adam.rs:52-95,162-197 and ghostflow-optim/src/sgd.rs:54-93.
"""
from __future__ import annotations

import torch

from . import _lib


def _gd(g: torch.Tensor) -> int:
    if g.dtype == torch.bfloat16:
        return 1
    if g.dtype == torch.float32:
        return 0
    raise TypeError(f"gradient dtype {g.dtype} not supported by the flat optimizer kernels")


def adam_flat(p, m, v, g, p_lp=None, *, lr, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.0, step=1,
              grad_scale=1.0, decoupled=True, skip_flag=None, step_dev=None):
    """In-place Adam/AdamW on fp32 ``p, m, v`` (1-D, contiguous) with gradient ``g`` (fp32 or bf16). ``step_dev``:
    int32 device tensor holding the step number (then ``step`` is ignored and the launch can be replayed from a
    CUDA graph)."""
    assert p.is_cuda and p.dtype == torch.float32 and p.is_contiguous()
    n = p.numel()
    rc = _lib.cuda_lib().gf_adam_flat_dev(
        p.data_ptr(), m.data_ptr(), v.data_ptr(), g.data_ptr(), p_lp.data_ptr() if p_lp is not None else None, n,
        float(lr), float(beta1), float(beta2), float(eps), float(weight_decay), int(step), float(grad_scale),
        1 if decoupled else 0, _gd(g), skip_flag.data_ptr() if skip_flag is not None else None,
        step_dev.data_ptr() if step_dev is not None else None, _lib.stream_ptr())
    _lib.check_rc(rc, "gf_adam_flat")


def sgd_flat(p, buf, g, p_lp=None, *, lr, momentum=0.0, dampening=0.0, weight_decay=0.0, nesterov=False,
             first_step=False, grad_scale=1.0):
    assert p.is_cuda and p.dtype == torch.float32 and p.is_contiguous()
    rc = _lib.cuda_lib().gf_sgd_flat(
        p.data_ptr(), buf.data_ptr() if buf is not None else None, g.data_ptr(),
        p_lp.data_ptr() if p_lp is not None else None, p.numel(), float(lr), float(momentum), float(dampening),
        float(weight_decay), 1 if nesterov else 0, 1 if first_step else 0, float(grad_scale), _gd(g),
        _lib.stream_ptr())
    _lib.check_rc(rc, "gf_sgd_flat")


def grad_sumsq(g: torch.Tensor, out: torch.Tensor) -> None:
    """Accumulates ``sum(g^2)`` into ``out[0]`` and raises ``out[1]`` to 1 when ``g`` has inf/nan."""
    rc = _lib.cuda_lib().gf_grad_sumsq(g.data_ptr(), g.numel(), out.data_ptr(), _gd(g), _lib.stream_ptr())
    _lib.check_rc(rc, "gf_grad_sumsq")
