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
