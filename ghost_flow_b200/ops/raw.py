"""Explicit forward / backward primitives (no autograd graph) used by the hand-scheduled training
engines. Each primitive launches the sm_100a kernel for bf16 CUDA tensors and runs the same math
in PyTorch for CPU tensors, so the engines' partitioning and scheduling logic can be tested with
CPU ranks over gloo.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F

from . import _lib
from .fused import _scratch, rope_ref
from .gemm import gemm_raw


def _k(t: torch.Tensor) -> bool:
    return t.is_cuda and t.dtype == torch.bfloat16


def _rc(rc, what):
    _lib.check_rc(rc, what)


# ------------------------------------------------------------------ GEMM
def gemm(a, a_t: bool, b, b_t: bool, out=None, out_dtype=None, bias=None, residual=None, accumulate=False,
         alpha=1.0, **kw):
    """``op(a) @ op(b)`` with ``op(a) = a^T`` when ``a_t`` (a stored [K, M]) and ``op(b) = b^T`` when
    ``b_t`` (b stored [N, K], the usual weight layout)."""
    M = a.shape[1] if a_t else a.shape[0]
    K = a.shape[0] if a_t else a.shape[1]
    N = b.shape[0] if b_t else b.shape[1]
    if _k(a) and _k(b):
        return gemm_raw(a, a_t, b, not b_t, M, N, K, out=out,
                        out_dtype=out_dtype or torch.bfloat16, bias=bias, residual=residual,
                        accumulate=accumulate, alpha=alpha, **kw)
    af = (a.t() if a_t else a).float()
    bf = (b.t() if b_t else b).float()
    y = alpha * (af @ bf)
    if bias is not None:
        y = y + bias.float()
    if residual is not None:
        y = y + residual.float()
    if out is not None:
        if accumulate:
            y = y + out.float()
        out.copy_(y.to(out.dtype))
        return out
    return y.to(out_dtype or a.dtype)


# ------------------------------------------------------------------ RMSNorm
def rmsnorm_fwd(x, w, eps, residual=None):
    """Returns (y, rstd, h) where h = x + residual (or x itself when there is no residual)."""
    T, D = x.shape
    if _k(x):
        y = torch.empty_like(x)
        rstd = torch.empty(T, dtype=torch.float32, device=x.device)
        h = torch.empty_like(x) if residual is not None else x
        _rc(_lib.cuda_lib().gf_rmsnorm_fwd(x.data_ptr(), residual.data_ptr() if residual is not None else None,
                                           w.data_ptr(), y.data_ptr(),
                                           h.data_ptr() if residual is not None else None, rstd.data_ptr(), T, D,
                                           float(eps), _lib.stream_ptr()), "gf_rmsnorm_fwd")
        return y, rstd, h
    h = x if residual is None else (x.float() + residual.float()).to(x.dtype)
    hf = h.float()
    rstd = torch.rsqrt(hf.pow(2).mean(-1) + eps)
    y = (hf * rstd[:, None] * w.float()).to(x.dtype)
    return y, rstd, h


def rmsnorm_bwd(x, w, dy, rstd, dres=None, dw_out=None):
    """Returns (dx, dw). ``dres`` is added into dx; ``dw_out`` receives dw when given."""
    T, D = x.shape
    if _k(x):
        dx = torch.empty_like(x)
        dw = dw_out if dw_out is not None else torch.empty_like(w)
        lib = _lib.cuda_lib()
        g = lib.gf_norm_bwd_grid(T)
        scratch = _scratch(x.device, g * D)
        _rc(lib.gf_rmsnorm_bwd(x.data_ptr(), w.data_ptr(), dy.data_ptr(), rstd.data_ptr(),
                               dres.data_ptr() if dres is not None else None, dx.data_ptr(), dw.data_ptr(),
                               scratch.data_ptr(), T, D, 0, _lib.stream_ptr()), "gf_rmsnorm_bwd")
        return dx, dw
    xf, gf, wf = x.float(), dy.float(), w.float()
    g = gf * wf
    r = rstd[:, None]
    dx = r * g - xf * (r ** 3) * (g * xf).mean(-1, keepdim=True)
    if dres is not None:
        dx = dx + dres.float()
    dw = (gf * xf * r).sum(0)
    if dw_out is not None:
        dw_out.copy_(dw.to(dw_out.dtype))
        dw = dw_out
    else:
        dw = dw.to(w.dtype)
    return dx.to(x.dtype), dw


# ------------------------------------------------------------------ RoPE (in place on [T, H, D] views)
def rope_(x3, cos, sin, S, interleaved=False, pos_offset=0, backward=False):
    T, H, D = x3.shape
    if _k(x3):
        _rc(_lib.cuda_lib().gf_rope(x3.data_ptr(), cos.data_ptr(), sin.data_ptr(), T, H, D, x3.stride(0),
                                    x3.stride(1), S, pos_offset, 1 if interleaved else 0, 1 if backward else 0,
                                    _lib.stream_ptr()), "gf_rope")
        return x3
    xb = x3.reshape(T // S, S, H, D)
    s = -sin if backward else sin
    x3.copy_(rope_ref(xb, cos, s, interleaved, pos_offset).reshape(T, H, D))
    return x3


# ------------------------------------------------------------------ SwiGLU
def swiglu_fwd(gu):
    T, F2 = gu.shape
    if _k(gu):
        y = torch.empty((T, F2 // 2), dtype=gu.dtype, device=gu.device)
        _rc(_lib.cuda_lib().gf_swiglu_fwd(gu.data_ptr(), y.data_ptr(), T, F2 // 2, _lib.stream_ptr()),
            "gf_swiglu_fwd")
        return y
    g, u = gu.float().chunk(2, -1)
    return (F.silu(g) * u).to(gu.dtype)


def swiglu_bwd(gu, dy, out=None):
    T, F2 = gu.shape
    if _k(gu):
        dgu = out if out is not None else torch.empty_like(gu)
        _rc(_lib.cuda_lib().gf_swiglu_bwd(gu.data_ptr(), dy.data_ptr(), dgu.data_ptr(), T, F2 // 2,
                                          _lib.stream_ptr()), "gf_swiglu_bwd")
        return dgu
    g, u = gu.float().chunk(2, -1)
    s = torch.sigmoid(g)
    d = dy.float()
    return torch.cat((d * u * (s + g * s * (1 - s)), d * g * s), -1).to(gu.dtype)


# ------------------------------------------------------------------ attention on packed rows
def attn_fwd(q, k, v, B, S, Hq, Hkv, D, causal=True, scale=None):
    """q: [B*S, Hq*D] view (row pitch free), k/v: [B*S, Hkv*D] views. Returns (o [B*S, Hq*D], lse [B,Hq,S])."""
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    if _k(q):
        o = torch.empty((B * S, Hq * D), dtype=q.dtype, device=q.device)
        lse = torch.empty((B, Hq, S), dtype=torch.float32, device=q.device)
        _rc(_lib.flash_fwd_fn()(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr(),
                                              B, S, Hq, Hkv, D, q.stride(0), k.stride(0), v.stride(0), Hq * D,
                                              float(scale), 1 if causal else 0,
                                              _lib.status_word(q.device).data_ptr(), _lib.stream_ptr()),
            "gf_flash_attn_fwd")
        return o, lse
    qf = q.float().reshape(B, S, Hq, D).transpose(1, 2)
    kf = k.float().reshape(B, S, Hkv, D).transpose(1, 2).repeat_interleave(Hq // Hkv, 1)
    vf = v.float().reshape(B, S, Hkv, D).transpose(1, 2).repeat_interleave(Hq // Hkv, 1)
    s = qf @ kf.transpose(-1, -2) * scale
    if causal:
        s = s.masked_fill(~torch.ones(S, S, dtype=torch.bool, device=q.device).tril(), float("-inf"))
    lse = torch.logsumexp(s, -1)
    o = (torch.softmax(s, -1) @ vf).transpose(1, 2).reshape(B * S, Hq * D).to(q.dtype)
    return o, lse


def attn_bwd(q, k, v, o, do, lse, dq, dk, dv, B, S, Hq, Hkv, D, causal=True, scale=None):
    """Writes dq/dk/dv (row-pitched views, e.g. slices of one packed dqkv buffer)."""
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    if _k(q):
        _lib.flash_attn_backward(q, k, v, o, do, lse, dq, dk, dv, B, S, Hq, Hkv, D,
                                 dict(q=q.stride(0), k=k.stride(0), v=v.stride(0), o=o.stride(0), do=do.stride(0),
                                      dq=dq.stride(0), dk=dk.stride(0), dv=dv.stride(0)), scale, causal)
        return
    G = Hq // Hkv
    qf = q.float().reshape(B, S, Hq, D).transpose(1, 2)
    kf = k.float().reshape(B, S, Hkv, D).transpose(1, 2).repeat_interleave(G, 1)
    vf = v.float().reshape(B, S, Hkv, D).transpose(1, 2).repeat_interleave(G, 1)
    dof = do.float().reshape(B, S, Hq, D).transpose(1, 2)
    s = qf @ kf.transpose(-1, -2) * scale
    if causal:
        s = s.masked_fill(~torch.ones(S, S, dtype=torch.bool, device=q.device).tril(), float("-inf"))
    # probabilities from the given log-sum-exp and delta from o, as in the kernel: k/v may be one block of a longer
    # key sequence (ring attention), in which case lse and o are those of the whole row
    p = torch.exp(s - lse.float().unsqueeze(-1))
    of = o.float().reshape(B, S, Hq, D).transpose(1, 2)
    dvf = p.transpose(-1, -2) @ dof
    dp = dof @ vf.transpose(-1, -2)
    ds = p * (dp - (dof * of).sum(-1, keepdim=True)) * scale
    dqf = ds @ kf
    dkf = ds.transpose(-1, -2) @ qf
    dkf = dkf.reshape(B, Hkv, G, S, D).sum(2)
    dvf = dvf.reshape(B, Hkv, G, S, D).sum(2)
    dq.copy_(dqf.transpose(1, 2).reshape(B * S, Hq * D).to(dq.dtype))
    dk.copy_(dkf.transpose(1, 2).reshape(B * S, Hkv * D).to(dk.dtype))
    dv.copy_(dvf.transpose(1, 2).reshape(B * S, Hkv * D).to(dv.dtype))


# ------------------------------------------------------------------ loss
def xent_fwd_bwd(logits, targets, grad_scale=None):
    """Mean cross-entropy; overwrites ``logits`` with d(loss)/d(logits). Returns the fp32 scalar loss tensor."""
    T, V = logits.shape
    scale = (1.0 / T) if grad_scale is None else grad_scale
    if _k(logits):
        loss_rows = torch.empty(T, dtype=torch.float32, device=logits.device)
        _rc(_lib.cuda_lib().gf_xent_fused(logits.data_ptr(), targets.data_ptr(), loss_rows.data_ptr(),
                                          logits.data_ptr(), T, V, logits.stride(0), float(scale), -(1 << 62),
                                          _lib.stream_ptr()), "gf_xent_fused")
        return loss_rows.sum() * scale
    lf = logits.float()
    lse = torch.logsumexp(lf, -1)
    loss_rows = lse - lf.gather(1, targets[:, None]).squeeze(1)
    p = torch.softmax(lf, -1)
    p[torch.arange(T), targets] -= 1.0
    logits.copy_((p * scale).to(logits.dtype))
    return loss_rows.sum() * scale


# ------------------------------------------------------------------ optimizer
def adamw_flat(p32, m, v, g, p_lp, *, lr, beta1, beta2, eps, weight_decay, step, grad_scale=1.0, decoupled=True):
    if p32.is_cuda:
        from .optim_kernels import adam_flat

        adam_flat(p32, m, v, g, p_lp, lr=lr, beta1=beta1, beta2=beta2, eps=eps, weight_decay=weight_decay,
                  step=step, grad_scale=grad_scale, decoupled=decoupled)
        return
    gf = g.float() * grad_scale
    if not decoupled:
        gf = gf + weight_decay * p32
    m.mul_(beta1).add_(gf, alpha=1 - beta1)
    v.mul_(beta2).addcmul_(gf, gf, value=1 - beta2)
    mh = m / (1 - beta1 ** step)
    vh = v / (1 - beta2 ** step)
    if decoupled:
        p32.mul_(1 - lr * weight_decay)
    p32.sub_(lr * mh / (vh.sqrt() + eps))
    if p_lp is not None:
        p_lp.copy_(p32.to(p_lp.dtype))


# ------------------------------------------------------------------ decode attention over a KV cache
def attn_decode(q, kcache, vcache, length, B, Hq, Hkv, D, scale=None, splits=None, out=None):
    """q [B, Hq * D]; caches [B, s_max, Hkv * D]; attends over the first ``length`` cache rows of every sequence
    (``length``: int, or an int32 tensor [B] of per-sequence lengths). Returns [B, Hq * D]."""
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    if _k(q):
        s_max = kcache.shape[1]
        per_seq = torch.is_tensor(length)
        n = s_max if per_seq else int(length)
        if splits is None:
            # enough CTAs for about eight per SM (the kernel hides DRAM latency with warps in flight), but no
            # slice shorter than 128 cache rows
            splits = max(1, min(32, -(-(148 * 8) // max(1, B * Hkv)), (n + 127) // 128))
        if out is None:
            out = torch.empty(B, Hq * D, dtype=q.dtype, device=q.device)
        scratch = torch.empty(B * Hq * splits * (D + 2), dtype=torch.float32, device=q.device)
        _rc(_lib.cuda_lib().gf_attn_decode(q.data_ptr(), q.stride(0), kcache.data_ptr(), vcache.data_ptr(), s_max,
                                           length.data_ptr() if per_seq else None, 0 if per_seq else n, out.data_ptr(),
                                           out.stride(0), B, Hq, Hkv, D, float(scale), splits, scratch.data_ptr(),
                                           _lib.stream_ptr()), "gf_attn_decode")
        return out
    G = Hq // Hkv
    res = torch.empty(B, Hq * D, dtype=q.dtype, device=q.device)
    for b in range(B):
        n = int(length[b]) if torch.is_tensor(length) else int(length)
        qf = q[b].float().view(Hkv, G, D)
        kf = kcache[b, :n].float().view(n, Hkv, D).permute(1, 0, 2)
        vf = vcache[b, :n].float().view(n, Hkv, D).permute(1, 0, 2)
        p = torch.softmax(qf @ kf.transpose(-1, -2) * scale, -1)
        res[b] = (p @ vf).reshape(Hq * D).to(q.dtype)
    if out is not None:
        out.copy_(res)
        return out
    return res
