"""Autograd functions over the hand-written sm_100a kernels: RMSNorm, LayerNorm, RoPE, SwiGLU,
GELU-family activations, softmax cross-entropy and FlashAttention.

Every function takes the CUDA path for bf16 CUDA tensors and a plain PyTorch fp32-capable path for
CPU tensors (used by the CPU configuration and the CPU test-suite). The PyTorch path is also the
numerical reference the GPU tests compare against.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F

from . import _lib

_SCRATCH = {}


def _scratch(device, nfloats: int) -> torch.Tensor:
    """Grow-only fp32 workspace per device (partial sums of the norm backward kernels)."""
    key = device.index if device.index is not None else torch.cuda.current_device()
    t = _SCRATCH.get(key)
    if t is None or t.numel() < nfloats:
        t = torch.empty(max(nfloats, 1 << 20), dtype=torch.float32, device=device)
        _SCRATCH[key] = t
    return t


def _cuda_bf16(*ts) -> bool:
    return all(t is None or (t.is_cuda and t.dtype == torch.bfloat16) for t in ts)


class _NoGraph:
    """Stand-in for the autograd context when nothing needs a gradient: the forward of an autograd function is then
    called directly, which skips the cost of creating a graph node (several microseconds per call on the host)."""

    needs_input_grad = ()

    def save_for_backward(self, *tensors):
        pass

    def mark_dirty(self, *tensors):
        pass


def _call(fn, *args):
    """``fn.apply(*args)`` when a gradient may be wanted, else ``fn.forward`` without a graph node."""
    if torch.is_grad_enabled():
        for a in args:
            if isinstance(a, torch.Tensor) and a.requires_grad:
                return fn.apply(*args)
    return fn.forward(_NoGraph(), *args)


def _rc(rc, what):
    _lib.check_rc(rc, what)
    if _lib.DEBUG_SYNC:
        _lib.check_status()


# ------------------------------------------------------------------------------------------ RMSNorm
class _RMSNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, eps, residual):
        D = x.shape[-1]
        x2 = x.reshape(-1, D).contiguous()
        T = x2.shape[0]
        y = torch.empty_like(x2)
        rstd = torch.empty(T, dtype=torch.float32, device=x.device)
        h = None
        res2 = None
        if residual is not None:
            res2 = residual.reshape(-1, D).contiguous()
            h = torch.empty_like(x2)
        lib = _lib.cuda_lib()
        _rc(lib.gf_rmsnorm_fwd(x2.data_ptr(), res2.data_ptr() if res2 is not None else None, w.data_ptr(),
                               y.data_ptr(), h.data_ptr() if h is not None else None, rstd.data_ptr(), T, D,
                               float(eps), _lib.stream_ptr()), "gf_rmsnorm_fwd")
        ctx.save_for_backward(h if h is not None else x2, w, rstd)
        ctx.shape = x.shape
        ctx.has_res = residual is not None
        if residual is not None:
            return y.view(x.shape), h.view(x.shape)
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy, dh=None):
        x2, w, rstd = ctx.saved_tensors
        T, D = x2.shape
        dy2 = dy.reshape(-1, D).contiguous()
        dres = dh.reshape(-1, D).contiguous() if (ctx.has_res and dh is not None) else None
        dx = torch.empty_like(x2)
        dw = torch.empty_like(w)
        lib = _lib.cuda_lib()
        g = lib.gf_norm_bwd_grid(T)
        scratch = _scratch(x2.device, g * D)
        _rc(lib.gf_rmsnorm_bwd(x2.data_ptr(), w.data_ptr(), dy2.data_ptr(), rstd.data_ptr(),
                               dres.data_ptr() if dres is not None else None, dx.data_ptr(), dw.data_ptr(),
                               scratch.data_ptr(), T, D, 0, _lib.stream_ptr()), "gf_rmsnorm_bwd")
        dxv = dx.view(ctx.shape)
        if ctx.has_res:
            return dxv, dw, None, dxv
        return dxv, dw, None, None


def rms_norm_ref(x, w, eps=1e-6):
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * w.float()
    return y.to(x.dtype)


def rms_norm(x, w, eps: float = 1e-6, residual=None):
    """RMSNorm; with ``residual`` returns ``(norm(x + residual), x + residual)`` from one kernel."""
    if _cuda_bf16(x, w, residual):
        return _call(_RMSNormFn, x, w, eps, residual)
    if residual is not None:
        h = x + residual
        return rms_norm_ref(h, w, eps), h
    return rms_norm_ref(x, w, eps)


# ------------------------------------------------------------------------------------------ LayerNorm
class _LayerNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, b, eps):
        D = x.shape[-1]
        x2 = x.reshape(-1, D).contiguous()
        T = x2.shape[0]
        y = torch.empty_like(x2)
        mean = torch.empty(T, dtype=torch.float32, device=x.device)
        rstd = torch.empty(T, dtype=torch.float32, device=x.device)
        lib = _lib.cuda_lib()
        _rc(lib.gf_layernorm_fwd(x2.data_ptr(), w.data_ptr(), b.data_ptr() if b is not None else None, y.data_ptr(),
                                 mean.data_ptr(), rstd.data_ptr(), T, D, float(eps), _lib.stream_ptr()),
            "gf_layernorm_fwd")
        ctx.save_for_backward(x2, w, mean, rstd)
        ctx.shape = x.shape
        ctx.has_bias = b is not None
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy):
        x2, w, mean, rstd = ctx.saved_tensors
        T, D = x2.shape
        dy2 = dy.reshape(-1, D).contiguous()
        dx = torch.empty_like(x2)
        dw = torch.empty_like(w)
        db = torch.empty_like(w) if ctx.has_bias else None
        lib = _lib.cuda_lib()
        g = lib.gf_norm_bwd_grid(T)
        scratch = _scratch(x2.device, 2 * g * D)
        _rc(lib.gf_layernorm_bwd(x2.data_ptr(), w.data_ptr(), dy2.data_ptr(), mean.data_ptr(), rstd.data_ptr(),
                                 dx.data_ptr(), dw.data_ptr(), db.data_ptr() if db is not None else None,
                                 scratch.data_ptr(), T, D, 0, _lib.stream_ptr()), "gf_layernorm_bwd")
        return dx.view(ctx.shape), dw, db, None


def layer_norm(x, w, b=None, eps: float = 1e-5):
    if _cuda_bf16(x, w, b) and x.shape[-1] % 8 == 0 and x.shape[-1] <= 8192:
        return _call(_LayerNormFn, x, w, b, eps)
    return F.layer_norm(x, (x.shape[-1],), w, b, eps)


# ------------------------------------------------------------------------------------------ RoPE
_ROPE_CACHE = {}


def rope_tables(seq_len: int, head_dim: int, theta: float = 10000.0, device="cpu"):
    """fp32 cos/sin tables ``[seq_len, head_dim/2]`` (angle = pos * theta^(-2i/d))."""
    key = (seq_len, head_dim, float(theta), str(device))
    t = _ROPE_CACHE.get(key)
    if t is None:
        inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float64) / head_dim))
        ang = torch.outer(torch.arange(seq_len, dtype=torch.float64), inv)
        t = (ang.cos().float().to(device).contiguous(), ang.sin().float().to(device).contiguous())
        _ROPE_CACHE[key] = t
    return t


def rope_ref(x, cos, sin, interleaved=False, pos_offset=0):
    """x: [..., S, H, D]; cos/sin: [>=S+pos_offset, D/2]."""
    S = x.shape[-3]
    c = cos[pos_offset:pos_offset + S].unsqueeze(-2).to(torch.float32)
    s = sin[pos_offset:pos_offset + S].unsqueeze(-2).to(torch.float32)
    xf = x.float()
    if interleaved:
        a, b = xf[..., 0::2], xf[..., 1::2]
        out = torch.stack((a * c - b * s, b * c + a * s), dim=-1).flatten(-2)
    else:
        h = x.shape[-1] // 2
        a, b = xf[..., :h], xf[..., h:]
        out = torch.cat((a * c - b * s, b * c + a * s), dim=-1)
    return out.to(x.dtype)


def _rope_launch(x, cos, sin, S, interleaved, pos_offset, backward):
    """In place on x viewed as [T, H, D] (unit stride over D; rows and heads may be strided)."""
    T, H, D = x.shape
    lib = _lib.cuda_lib()
    _rc(lib.gf_rope(x.data_ptr(), cos.data_ptr(), sin.data_ptr(), T, H, D, x.stride(0), x.stride(1), S, pos_offset,
                    1 if interleaved else 0, 1 if backward else 0, _lib.stream_ptr()), "gf_rope")


class _RopeFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, cos, sin, interleaved, pos_offset, inplace):
        # x: [B, S, H, D] (any row/head strides)
        B, S, H, D = x.shape
        out = x if inplace else x.clone()
        v = out.view(B * S, H, D) if out.is_contiguous() else out.reshape(B * S, H, D)
        if v.data_ptr() != out.data_ptr() or v.stride(2) != 1:
            raise RuntimeError("rope needs a [B,S,H,D] tensor whose (B,S) dims can be flattened without a copy")
        _rope_launch(v, cos, sin, S, interleaved, pos_offset, False)
        ctx.save_for_backward(cos, sin)
        ctx.args = (S, interleaved, pos_offset)
        if inplace:
            ctx.mark_dirty(x)
        return out

    @staticmethod
    def backward(ctx, dy):
        cos, sin = ctx.saved_tensors
        S, interleaved, pos_offset = ctx.args
        g = dy.contiguous().clone()
        B, S_, H, D = g.shape
        _rope_launch(g.view(B * S_, H, D), cos, sin, S, interleaved, pos_offset, True)
        return g, None, None, None, None, None


def rope(x, cos, sin, interleaved: bool = False, pos_offset: int = 0, inplace: bool = False):
    """Rotary embedding on ``[B, S, H, D]``; half-split pairing by default, ``interleaved`` for (2i, 2i+1)."""
    if x.is_cuda and x.dtype == torch.bfloat16 and x.shape[-1] % 16 == 0:
        return _call(_RopeFn, x, cos, sin, interleaved, pos_offset, inplace)
    return rope_ref(x, cos, sin, interleaved, pos_offset)


# ------------------------------------------------------------------------------------------ SwiGLU / unary
class _SwiGLUFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gu):
        F2 = gu.shape[-1]
        g2 = gu.reshape(-1, F2).contiguous()
        T = g2.shape[0]
        y = torch.empty((T, F2 // 2), dtype=gu.dtype, device=gu.device)
        _rc(_lib.cuda_lib().gf_swiglu_fwd(g2.data_ptr(), y.data_ptr(), T, F2 // 2, _lib.stream_ptr()),
            "gf_swiglu_fwd")
        ctx.save_for_backward(g2)
        ctx.shape = gu.shape
        return y.view(*gu.shape[:-1], F2 // 2)

    @staticmethod
    def backward(ctx, dy):
        (g2,) = ctx.saved_tensors
        T, F2 = g2.shape
        dy2 = dy.reshape(T, F2 // 2).contiguous()
        dgu = torch.empty_like(g2)
        _rc(_lib.cuda_lib().gf_swiglu_bwd(g2.data_ptr(), dy2.data_ptr(), dgu.data_ptr(), T, F2 // 2,
                                          _lib.stream_ptr()), "gf_swiglu_bwd")
        return dgu.view(ctx.shape)


def swiglu(gu):
    """``silu(gate) * up`` where ``gu = [..., gate | up]`` is the fused gate/up projection output."""
    if _cuda_bf16(gu) and (gu.shape[-1] // 2) % 8 == 0:
        return _call(_SwiGLUFn, gu)
    g, u = gu.chunk(2, dim=-1)
    return F.silu(g) * u


OPS = {"relu": 0, "gelu": 1, "sigmoid": 2, "tanh": 3, "silu": 4}


class _UnaryFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, op):
        xc = x.contiguous()
        y = torch.empty_like(xc)
        _rc(_lib.cuda_lib().gf_unary_fwd(xc.data_ptr(), y.data_ptr(), xc.numel(), op, 1, _lib.stream_ptr()),
            "gf_unary_fwd")
        ctx.save_for_backward(xc)
        ctx.op = op
        return y

    @staticmethod
    def backward(ctx, dy):
        (xc,) = ctx.saved_tensors
        dyc = dy.contiguous()
        dx = torch.empty_like(xc)
        _rc(_lib.cuda_lib().gf_unary_bwd_bf16(xc.data_ptr(), dyc.data_ptr(), dx.data_ptr(), xc.numel(), ctx.op,
                                              _lib.stream_ptr()), "gf_unary_bwd_bf16")
        return dx, None


def _unary_ref(x, name):
    if name == "relu":
        return torch.relu(x)
    if name == "gelu":
        return F.gelu(x, approximate="tanh")
    if name == "sigmoid":
        return torch.sigmoid(x)
    if name == "tanh":
        return torch.tanh(x)
    return F.silu(x)


def unary(x, name: str):
    """relu / gelu (tanh form) / sigmoid / tanh / silu."""
    if _cuda_bf16(x) and x.numel() % 8 == 0 and x.numel() > 0:
        return _call(_UnaryFn, x, OPS[name])
    return _unary_ref(x, name)


def gelu(x):
    return unary(x, "gelu")


def op_chain(x, names):
    """Applies a chain of unary ops in one pass over memory (inference helper, no autograd)."""
    if x.is_cuda and x.dtype in (torch.bfloat16, torch.float32) and len(names) <= 8:
        import ctypes

        xc = x.contiguous()
        y = torch.empty_like(xc)
        arr = (ctypes.c_int * len(names))(*[OPS[n] for n in names])
        _rc(_lib.cuda_lib().gf_op_chain(xc.data_ptr(), y.data_ptr(), xc.numel(), arr, len(names),
                                        1 if x.dtype == torch.bfloat16 else 0, _lib.stream_ptr()), "gf_op_chain")
        return y
    for n in names:
        x = _unary_ref(x, n)
    return x


# ------------------------------------------------------------------------------------------ cross-entropy
def _padded_rows(rows: int, cols: int, device, dtype, pitch: int | None = None) -> torch.Tensor:
    """``[rows, cols]`` view of a buffer whose row pitch is a multiple of 64 elements: every row starts on a 16-byte
    boundary whatever ``cols`` is (a 50257-column logits matrix would not otherwise), which is what TMA tensor maps
    and the vectorised row kernels need. The padding columns are not initialised."""
    pitch = pitch or (cols + 63) // 64 * 64
    return torch.empty(rows, pitch, device=device, dtype=dtype)[:, :cols]


class _XentFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, targets, ignore_index, inplace_grad):
        V = logits.shape[-1]
        l2 = logits.reshape(-1, V)
        if l2.stride(-1) != 1 or l2.stride(0) % 8 or l2.stride(0) < (V + 7) // 8 * 8 or l2.data_ptr() % 16:
            # rows must start on 16-byte boundaries and leave room for the last vector: copy into a padded buffer
            l2 = _padded_rows(l2.shape[0], V, l2.device, l2.dtype).copy_(l2)
        T = l2.shape[0]
        tg = targets.reshape(-1).to(torch.int64).contiguous()
        n_valid = None
        if ignore_index is not None:
            n_valid = (tg != ignore_index).sum().clamp(min=1).to(torch.float32)
        loss_rows = torch.empty(T, dtype=torch.float32, device=logits.device)
        need_grad = logits.requires_grad
        dl = None
        if need_grad:
            dl = l2 if inplace_grad else _padded_rows(T, V, l2.device, l2.dtype, pitch=l2.stride(0))
        # the 1/N of the mean is folded in here; backward only multiplies by the incoming scalar
        scale = 1.0 / T if n_valid is None else None
        if scale is None:
            scale = 1.0 / float(n_valid.item())
        _rc(_lib.cuda_lib().gf_xent_fused(l2.data_ptr(), tg.data_ptr(), loss_rows.data_ptr(),
                                          dl.data_ptr() if dl is not None else None, T, V, l2.stride(0), scale,
                                          ignore_index if ignore_index is not None else -(1 << 62),
                                          _lib.stream_ptr()), "gf_xent_fused")
        loss = loss_rows.sum() * scale
        ctx.save_for_backward(dl if dl is not None else torch.empty(0, device=logits.device))
        ctx.shape = logits.shape
        return loss

    @staticmethod
    def backward(ctx, dloss):
        (dl,) = ctx.saved_tensors
        if dl.numel() == 0:
            return None, None, None, None
        g = dl.view(ctx.shape)
        # dloss is 1.0 for a plain loss.backward(): scale only when it is something else. On the GPU the kernel
        # reads the scalar and returns at once when it is 1, so the host never waits for the value (a host read
        # here would stall every backward pass and cannot be recorded in a CUDA graph).
        if dloss.numel() != 1:
            return g * dloss.to(g.dtype), None, None, None
        g2 = g.reshape(-1, g.shape[-1])
        if g.is_cuda and g.dtype == torch.bfloat16 and g2.stride(1) == 1 and g2.data_ptr() == g.data_ptr() \
                and g.data_ptr() % 16 == 0:
            # rows may have a padded pitch: the span from the first to the last element is scaled, padding included
            span = (g2.shape[0] - 1) * g2.stride(0) + g2.shape[1]
            _lib.check_rc(_lib.cuda_lib().gf_scale_by_dev_scalar(g.data_ptr(), span,
                                                                 dloss.float().data_ptr(), _lib.stream_ptr()),
                          "gf_scale_by_dev_scalar")
            return g, None, None, None
        return (g * dloss.to(g.dtype) if float(dloss) != 1.0 else g), None, None, None


def cross_entropy(logits, targets, ignore_index: int | None = None, inplace_grad: bool = False):
    """Mean softmax cross-entropy over rows. On CUDA bf16 the forward also produces the logits
    gradient in the same pass (``inplace_grad=True`` overwrites ``logits`` with it).
    ``ignore_index=None`` promises that every target is a class id, which avoids a host sync."""
    V = logits.shape[-1]
    if _cuda_bf16(logits) and (V + 7) // 8 * 16 <= 200 * 1024:
        return _XentFn.apply(logits, targets, ignore_index, inplace_grad)
    return F.cross_entropy(logits.reshape(-1, V).float(), targets.reshape(-1).long(),
                           ignore_index=-100 if ignore_index is None else ignore_index)


# ------------------------------------------------------------------------------------------ attention
def attention_ref(q, k, v, causal=True, scale=None):
    """fp32 reference SDPA. q: [B,S,Hq,D]; k, v: [B,S,Hkv,D]."""
    B, S, Hq, D = q.shape
    Hkv = k.shape[2]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    qf = q.float().transpose(1, 2)
    kf = k.float().transpose(1, 2).repeat_interleave(Hq // Hkv, dim=1)
    vf = v.float().transpose(1, 2).repeat_interleave(Hq // Hkv, dim=1)
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    if causal:
        mask = torch.ones(S, k.shape[1], dtype=torch.bool, device=q.device).tril()
        s = s.masked_fill(~mask, float("-inf"))
    p = torch.softmax(s, dim=-1)
    return torch.matmul(p, vf).transpose(1, 2).to(q.dtype)


def _rows_view(t):
    """[B,S,H,D] -> (2-D alias [B*S, H*D] pitch) requirements: unit stride over D, heads packed."""
    B, S, H, D = t.shape
    if t.stride(3) != 1 or t.stride(2) != D or t.stride(0) != S * t.stride(1):
        return None
    return t.stride(1)


class _FlashAttnFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, causal, scale):
        B, S, Hq, D = q.shape
        Hkv = k.shape[2]
        ldq, ldk, ldv = _rows_view(q), _rows_view(k), _rows_view(v)
        if ldq is None or (ldq % 8):
            q = q.contiguous(); ldq = Hq * D
        if ldk is None or (ldk % 8):
            k = k.contiguous(); ldk = Hkv * D
        if ldv is None or (ldv % 8):
            v = v.contiguous(); ldv = Hkv * D
        o = torch.empty((B, S, Hq, D), dtype=q.dtype, device=q.device)
        lse = torch.empty((B, Hq, S), dtype=torch.float32, device=q.device)
        lib = _lib.cuda_lib()
        _rc(_lib.flash_fwd_fn()(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr(), B, S, Hq,
                                  Hkv, D, ldq, ldk, ldv, Hq * D, float(scale), 1 if causal else 0,
                                  _lib.status_word(q.device).data_ptr(), _lib.stream_ptr()), "gf_flash_attn_fwd")
        ctx.save_for_backward(q, k, v, o, lse)
        ctx.args = (causal, scale, ldq, ldk, ldv)
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, o, lse = ctx.saved_tensors
        causal, scale, ldq, ldk, ldv = ctx.args
        B, S, Hq, D = q.shape
        Hkv = k.shape[2]
        if S % 128:
            raise RuntimeError("flash attention backward needs a sequence length that is a multiple of 128")
        do = do.contiguous()
        # one packed gradient buffer [B,S,(Hq+2Hkv),D] so a fused QKV projection sees a single tensor
        dqkv = torch.empty((B, S, Hq + 2 * Hkv, D), dtype=q.dtype, device=q.device)
        dq, dk, dv = dqkv[:, :, :Hq], dqkv[:, :, Hq:Hq + Hkv], dqkv[:, :, Hq + Hkv:]
        ldg = (Hq + 2 * Hkv) * D
        _lib.flash_attn_backward(q, k, v, o, do, lse, dq, dk, dv, B, S, Hq, Hkv, D,
                                 dict(q=ldq, k=ldk, v=ldv, o=Hq * D, do=Hq * D, dq=ldg, dk=ldg, dv=ldg), scale, causal)
        return dq, dk, dv, None, None


class _SplitQKVFn(torch.autograd.Function):
    """``qkv [B, S, H + 2 Hk, D] -> q, k, v`` as views. Plain slicing gives the same forward, but its backward pads
    each of the three gradients to the full shape with zeros and adds them (six passes over the packed tensor); the
    attention backward already writes its three gradients into one packed buffer, which this function recognises
    and hands on as it is."""

    @staticmethod
    def forward(ctx, qkv, H, Hk):
        ctx.H, ctx.Hk = H, Hk
        return qkv[:, :, :H], qkv[:, :, H:H + Hk], qkv[:, :, H + Hk:]

    @staticmethod
    def backward(ctx, dq, dk, dv):
        H, Hk = ctx.H, ctx.Hk
        if dq is None or dk is None or dv is None:
            ref = next(t for t in (dq, dk, dv) if t is not None)
            B, S, _, D = ref.shape
            dq = dq if dq is not None else ref.new_zeros(B, S, H, D)
            dk = dk if dk is not None else ref.new_zeros(B, S, Hk, D)
            dv = dv if dv is not None else ref.new_zeros(B, S, Hk, D)
        B, S, _, D = dq.shape
        G = H + 2 * Hk
        packed = (S * G * D, G * D, D, 1)
        same = (dq.untyped_storage().data_ptr() == dk.untyped_storage().data_ptr() == dv.untyped_storage().data_ptr()
                and dq.stride() == packed and dk.stride() == packed and dv.stride() == packed
                and dk.storage_offset() == dq.storage_offset() + H * D
                and dv.storage_offset() == dq.storage_offset() + (H + Hk) * D)
        if same:
            return dq.as_strided((B, S, G, D), packed, dq.storage_offset()), None, None
        return torch.cat((dq, dk, dv), 2), None, None


def split_qkv(qkv: torch.Tensor, num_heads: int, num_kv_heads: int):
    """Views ``q [B,S,H,D]``, ``k``, ``v [B,S,Hk,D]`` of a packed projection output ``[B,S,H+2Hk,D]``."""
    if torch.is_grad_enabled() and qkv.requires_grad:
        return _SplitQKVFn.apply(qkv, num_heads, num_kv_heads)
    H, Hk = num_heads, num_kv_heads
    return qkv[:, :, :H], qkv[:, :, H:H + Hk], qkv[:, :, H + Hk:]


def flash_attention(q, k, v, causal: bool = True, scale: float | None = None):
    """Attention over ``q [B,S,Hq,D]``, ``k/v [B,S,Hkv,D]`` (views into a packed QKV tensor are fine).
    head_dim 64 or 128 on the tcgen05 kernels; anything else uses the fp32 reference math."""
    D = q.shape[-1]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    if _cuda_bf16(q, k, v) and D in (64, 128) and q.shape[1] == k.shape[1]:
        return _call(_FlashAttnFn, q, k, v, causal, scale)
    return attention_ref(q, k, v, causal, scale)
