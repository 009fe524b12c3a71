"""fp8 (e4m3) quantisation and the scaled fp8 GEMM.

The reference only rounds fp32 values to an fp8 grid (ghostflow-nn/src/mixed_precision.rs:264-285, "fake fp8");
here operands are stored as e4m3 bytes and multiplied on the tensor cores.

Two schemes (``mode``):

* ``0`` per-row scales: one scale per token for activations, one per output channel for weights.
* ``1`` block scales: 1 x 128 blocks for activations (scale stored ``[K / 128, T]``), 128 x 128 blocks for weights
  (scale ``[ceil(N / 128), K / 128]``).

Every function has a PyTorch path for CPU tensors that produces the same bytes and scales (the test oracle).
"""
from __future__ import annotations

import ctypes

import torch

from . import _lib

E4M3_MAX = 448.0
_BOUND = False


def _bind():
    global _BOUND
    lib = _lib.cuda_lib()
    if not _BOUND:
        P, I, L = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong
        lib.gf_quant_fp8_rows.argtypes = [P, L, P, L, P, I, I, I, P]
        lib.gf_quant_fp8_block128.argtypes = [P, L, P, L, P, I, I, P]
        lib.gf_gemm_fp8.argtypes = [P, P, P, I, I, I, L, L, L, P, P, P, I, P, P]
        for n in ("gf_quant_fp8_rows", "gf_quant_fp8_block128", "gf_gemm_fp8"):
            getattr(lib, n).restype = I
        _BOUND = True
    return lib


def quantize_rows(x: torch.Tensor, mode: int = 0):
    """x [T, K] bf16 -> (q uint8 [T, K] holding e4m3 bytes, scale fp32: [T] (mode 0) or [K / 128, T] (mode 1))."""
    T, K = x.shape
    if x.is_cuda:
        x = x.contiguous()
        q = torch.empty(T, K, dtype=torch.uint8, device=x.device)
        scale = torch.empty(T if mode == 0 else (K // 128, T), dtype=torch.float32, device=x.device)
        _lib.check_rc(_bind().gf_quant_fp8_rows(x.data_ptr(), x.stride(0), q.data_ptr(), q.stride(0), scale.data_ptr(),
                                                T, K, mode, _lib.stream_ptr()), "gf_quant_fp8_rows")
        return q, scale
    xf = x.float()
    if mode == 0:
        s = xf.abs().amax(1).clamp_min(1e-12) / E4M3_MAX
        q = (xf / s[:, None]).clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn).view(torch.uint8)
        return q, s
    xb = xf.view(T, K // 128, 128)
    s = xb.abs().amax(2).clamp_min(1e-12) / E4M3_MAX
    q = (xb / s[:, :, None]).clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn).view(torch.uint8).view(T, K)
    return q, s.t().contiguous()


def quantize_block128(w: torch.Tensor):
    """w [N, K] bf16 -> (q uint8 [N, K], scale fp32 [ceil(N / 128), K / 128])."""
    N, K = w.shape
    nb, kb = (N + 127) // 128, K // 128
    if w.is_cuda:
        w = w.contiguous()
        q = torch.empty(N, K, dtype=torch.uint8, device=w.device)
        scale = torch.empty(nb, kb, dtype=torch.float32, device=w.device)
        _lib.check_rc(_bind().gf_quant_fp8_block128(w.data_ptr(), w.stride(0), q.data_ptr(), q.stride(0),
                                                    scale.data_ptr(), N, K, _lib.stream_ptr()), "gf_quant_fp8_block128")
        return q, scale
    wf = torch.zeros(nb * 128, K)
    wf[:N] = w.float()
    blocks = wf.view(nb, 128, kb, 128)
    s = blocks.abs().amax((1, 3)).clamp_min(1e-12) / E4M3_MAX
    q = (blocks / s[:, None, :, None]).clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn).view(torch.uint8)
    return q.view(nb * 128, K)[:N].contiguous(), s


def dequantize(q: torch.Tensor, scale: torch.Tensor, mode: int, weight: bool = False) -> torch.Tensor:
    """fp32 values represented by (q, scale)."""
    v = q.view(torch.float8_e4m3fn).float()
    R, K = v.shape
    if mode == 0:
        return v * scale[:, None]
    if weight:
        s = scale.repeat_interleave(128, 0)[:R].repeat_interleave(128, 1)
        return v * s
    return v * scale.t().repeat_interleave(128, 1)


def gemm_fp8(aq, sa, bq, sb, mode: int = 0, bias=None, out=None) -> torch.Tensor:
    """``out[M, N] (bf16) = dequant(aq, sa) @ dequant(bq, sb)^T`` with aq [M, K], bq [N, K] e4m3 bytes."""
    M, K = aq.shape
    N = bq.shape[0]
    if aq.is_cuda:
        if out is None:
            out = torch.empty(M, N, dtype=torch.bfloat16, device=aq.device)
        rc = _bind().gf_gemm_fp8(aq.data_ptr(), bq.data_ptr(), out.data_ptr(), M, N, K, aq.stride(0), bq.stride(0),
                                 out.stride(0), sa.data_ptr(), sb.data_ptr(), bias.data_ptr() if bias is not None else None,
                                 mode, _lib.status_word(aq.device).data_ptr(), _lib.stream_ptr())
        _lib.check_rc(rc, "gf_gemm_fp8")
        return out
    y = dequantize(aq, sa, mode) @ dequantize(bq, sb, mode, weight=True).t()
    if bias is not None:
        y = y + bias.float()
    y = y.to(torch.bfloat16)
    if out is not None:
        out.copy_(y)
        return out
    return y


class Fp8Linear(torch.nn.Module):
    """Inference linear layer with e4m3 weights quantised once and activations quantised per call."""

    def __init__(self, weight: torch.Tensor, bias: torch.Tensor | None = None, mode: int = 0):
        super().__init__()
        self.mode = mode
        if mode == 0:
            q, s = quantize_rows(weight.to(torch.bfloat16), 0)
        else:
            q, s = quantize_block128(weight.to(torch.bfloat16))
        self.register_buffer("qweight", q)
        self.register_buffer("scale", s)
        self.bias = bias
        self.out_features, self.in_features = weight.shape

    @torch.no_grad()
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        shape = x.shape
        x2 = x.reshape(-1, shape[-1]).to(torch.bfloat16)
        xq, xs = quantize_rows(x2, self.mode)
        y = gemm_fp8(xq, xs, self.qweight, self.scale, self.mode, self.bias)
        return y.view(*shape[:-1], self.out_features)


# ------------------------------------------------------------------------------------------ training linear
class _Fp8LinearFn(torch.autograd.Function):
    """``y = x @ w^T (+ bias)`` with all three products of the layer (forward, input gradient, weight gradient) on
    the e4m3 tensor-core kernel. Every operand of every product is quantised along its own contraction axis with one
    scale per row (``quantize_rows`` of the operand, transposed where the contraction runs over its rows):

    * forward   ``y[T,N]  = q(x)[T,K]   . q(w)[N,K]^T``    scales per token and per output feature
    * dgrad     ``dx[T,K] = q(dy)[T,N]  . q(w^T)[K,N]^T``  scales per token and per input feature
    * wgrad     ``dw[N,K] = q(dy^T)[N,T]. q(x^T)[K,T]^T``  scales per output feature and per input feature

    Accumulation is fp32 in tensor memory; results are bf16. The bf16 master weight stays the parameter: nothing is
    kept in fp8 between steps (the reference's fp8 mode is likewise a cast around fp32 state,
    ghostflow-nn/src/mixed_precision.rs:29-60, 264-285)."""

    @staticmethod
    def forward(ctx, x, w, bias):
        x2 = x.reshape(-1, x.shape[-1]).to(torch.bfloat16)
        wq, ws = quantize_rows(w.to(torch.bfloat16), 0)
        xq, xs = quantize_rows(x2, 0)
        y = gemm_fp8(xq, xs, wq, ws, 0, bias)
        ctx.save_for_backward(x2, w)
        ctx.has_bias = bias is not None
        ctx.x_shape, ctx.x_dtype = x.shape, x.dtype
        return y.view(*x.shape[:-1], w.shape[0]).to(x.dtype)

    @staticmethod
    def backward(ctx, dy):
        x2, w = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1]).to(torch.bfloat16)
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            gq, gs = quantize_rows(dy2.contiguous(), 0)
            wtq, wts = quantize_rows(w.to(torch.bfloat16).t().contiguous(), 0)
            dx = gemm_fp8(gq, gs, wtq, wts, 0).view(ctx.x_shape).to(ctx.x_dtype)
        if ctx.needs_input_grad[1]:
            gtq, gts = quantize_rows(dy2.t().contiguous(), 0)
            xtq, xts = quantize_rows(x2.t().contiguous(), 0)
            dw = gemm_fp8(gtq, gts, xtq, xts, 0).to(w.dtype)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = dy2.float().sum(0).to(dy.dtype)
        return dx, dw, db


def fp8_linear(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
    """Differentiable linear layer whose three GEMMs run in e4m3 (see :class:`_Fp8LinearFn`). The contraction
    lengths (in-features, out-features, tokens) must be multiples of 16 on the GPU kernel."""
    return _Fp8LinearFn.apply(x, w, bias)


class Fp8TrainLinear(torch.nn.Linear):
    """Drop-in ``nn.Linear`` whose forward and backward products are e4m3 GEMMs; parameters stay bf16 / fp32."""

    def forward(self, x):
        return fp8_linear(x, self.weight, self.bias)


def convert_linears_to_fp8(module: torch.nn.Module, skip=("lm_head",)) -> int:
    """Replaces every ``torch.nn.Linear`` (and subclass using ``weight`` / ``bias``) below ``module`` whose name is
    not in ``skip`` by :class:`Fp8TrainLinear` sharing the same parameters. Returns the number of layers converted."""
    n = 0
    for name, child in list(module.named_children()):
        if isinstance(child, torch.nn.Linear) and not isinstance(child, Fp8TrainLinear) and name not in skip:
            new = Fp8TrainLinear(child.in_features, child.out_features, child.bias is not None,
                                 device=child.weight.device, dtype=child.weight.dtype)
            new.weight, new.bias = child.weight, child.bias
            setattr(module, name, new)
            n += 1
        else:
            n += convert_linears_to_fp8(child, skip)
    return n


# ------------------------------------------------------------------------------------------ MX (block-scaled) format
# OCP microscaling MXFP8: blocks of 32 consecutive elements along the contraction axis share one power-of-two scale
# stored as E8M0 (a biased exponent byte, value 2^(e - 127)); the elements are e4m3. This is the operand format of
# `tcgen05.mma.kind::mxf8f6f4.block_scale`. The quantiser, the de-quantiser and the fp32 oracle below define the format
# for this package and are what a native block-scaled kernel has to reproduce; the GEMM entry point here runs the
# de-quantised operands through the bf16 tensor-core kernel (exact for the scales, bf16 rounding for the products of
# two e4m3 values is exact too: 4 + 4 significant bits), so it is a correct but not a native MX path.
MX_BLOCK = 32
_E4M3_EMAX = 8          # largest power of two representable in e4m3 (448 = 1.75 * 2^8)


def quantize_mxfp8(x: torch.Tensor):
    """``x [R, K]`` (K a multiple of 32) -> ``(q uint8 [R, K]`` e4m3 bytes, ``scale uint8 [R, K / 32]`` E8M0 bytes)``.
    The shared exponent of a block is ``floor(log2(amax)) - 8`` as the OCP specification prescribes."""
    R, K = x.shape
    assert K % MX_BLOCK == 0, "the contraction length must be a multiple of 32"
    xb = x.float().reshape(R, K // MX_BLOCK, MX_BLOCK)
    amax = xb.abs().amax(-1)
    e = torch.floor(torch.log2(amax.clamp_min(2.0 ** -126))) - _E4M3_EMAX
    e = e.clamp(-127, 127)
    scale = torch.exp2(e)
    q = (xb / scale[..., None]).clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn).view(torch.uint8).reshape(R, K)
    return q, (e + 127).to(torch.uint8)


def dequantize_mxfp8(q: torch.Tensor, scale_e8m0: torch.Tensor) -> torch.Tensor:
    """fp32 values of an MXFP8 tensor."""
    R, K = q.shape
    v = q.view(torch.float8_e4m3fn).float().reshape(R, K // MX_BLOCK, MX_BLOCK)
    s = torch.exp2(scale_e8m0.float() - 127.0)
    return (v * s[..., None]).reshape(R, K)


def gemm_mxfp8(aq, sa, bq, sb, out_dtype=torch.bfloat16) -> torch.Tensor:
    """``out[M, N] = dequant(aq, sa) @ dequant(bq, sb)^T`` for MXFP8 operands ``aq [M, K]``, ``bq [N, K]``.
    CPU: fp32 oracle. CUDA: the de-quantised operands through the bf16 tensor-core GEMM (see the note above)."""
    a, b = dequantize_mxfp8(aq, sa), dequantize_mxfp8(bq, sb)
    if aq.is_cuda:
        from . import gemm as _gemm

        return _gemm.matmul_nt(a.to(torch.bfloat16), b.to(torch.bfloat16)).to(out_dtype)
    return (a @ b.t()).to(out_dtype)
