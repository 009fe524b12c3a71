"""bf16 GEMM on the hand-written tcgen05 kernel, plus the ``linear`` autograd function.

On CUDA bf16 tensors every product (forward, dgrad, wgrad) runs ``gf_gemm_bf16``; CPU tensors
(the CPU configs and the CPU-only tests) use ``torch.matmul``. Other CUDA dtypes go to the
vendor GEMM as a plain library call.

Reference counterparts: ``ghostflow-core/src/ops/matmul.rs:13-170`` (CPU blocked matmul),
``ghostflow-cuda/src/blas.rs:278-313`` (cuBLAS row-major trick), ``ghostflow-nn/src/linear.rs:56-69``.
"""
from __future__ import annotations

import torch

from . import _lib


_SMS: dict = {}


def _sm_count(device) -> int:
    i = device.index if device.index is not None else torch.cuda.current_device()
    if i not in _SMS:
        _SMS[i] = torch.cuda.get_device_properties(i).multi_processor_count
    return _SMS[i]


def _is_dense_2d(t: torch.Tensor) -> bool:
    return t.dim() == 2 and t.stride(1) == 1 and t.stride(0) >= t.size(1)


def gemm_raw(a, a_mn_major, b, b_mn_major, M, N, K, out=None, out_dtype=torch.bfloat16, bias=None, residual=None,
             accumulate=False, alpha=1.0, bn_hint=0, max_ctas=0, relu=False):
    """Launches the kernel on 2-D row-major views.

    ``a`` is stored ``[M, K]`` (K-major) or ``[K, M]`` when ``a_mn_major``; ``b`` is stored
    ``[N, K]`` or ``[K, N]`` when ``b_mn_major``. Row pitches may exceed the row length. ``relu`` applies
    max(., 0) in the epilogue after bias and residual.
    """
    assert a.is_cuda and a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16
    assert _is_dense_2d(a) and _is_dense_2d(b), "operands must be 2-D with unit inner stride"
    if out is None:
        if N % 8:
            # rows of an [M, N] tensor with such an N do not start on 16-byte boundaries; give the result a padded
            # pitch (the caller gets an [M, N] view) so that it can feed the next kernel as it is
            out = torch.empty((M, (N + 63) // 64 * 64), dtype=out_dtype, device=a.device)[:, :N]
        else:
            out = torch.empty((M, N), dtype=out_dtype, device=a.device)
    assert _is_dense_2d(out)
    lib = _lib.cuda_lib()
    # few output tiles and a long K: the kernel splits K and needs an fp32 [M, N] workspace. It comes from torch's
    # allocator, so it belongs to the current stream (and to the graph's pool while a CUDA graph is recorded).
    ws = None
    if (K >= 2048 and out.dtype == torch.bfloat16 and not accumulate and not relu and bn_hint == 0 and max_ctas == 0
            and M * N < (1 << 31)
            and 2 * ((M + 127) // 128) * ((N + (127 if N <= 128 else 255)) // (128 if N <= 128 else 256)) <= _sm_count(a.device)):
        ws = torch.empty(M * N, dtype=torch.float32, device=a.device)
    rc = lib.gf_gemm_bf16(
        a.data_ptr(), b.data_ptr(), out.data_ptr(), M, N, K,
        1 if a_mn_major else 0, a.stride(0), 1 if b_mn_major else 0, b.stride(0), out.stride(0),
        1 if out.dtype == torch.float32 else 0, 1 if accumulate else 0,
        bias.data_ptr() if bias is not None else None,
        residual.data_ptr() if residual is not None else None,
        residual.stride(0) if residual is not None else 0,
        float(alpha), _lib.status_word(a.device).data_ptr(), bn_hint, max_ctas,
        ws.data_ptr() if ws is not None else None, 1 if relu else 0, ws.numel() if ws is not None else 0,
        _lib.stream_ptr(),
    )
    _lib.check_rc(rc, "gf_gemm_bf16")
    if _lib.DEBUG_SYNC:
        _lib.check_status(a.device)
    return out


def _kernel_ok(*ts) -> bool:
    """bf16 CUDA operands whose 2-D view satisfies the TMA rules (16-byte base and row pitch)."""
    for t in ts:
        if not (t.is_cuda and t.dtype == torch.bfloat16):
            return False
        if t.dim() >= 2 and (t.stride(-1) != 1 or (t.stride(-2) % 8) or (t.data_ptr() % 16)):
            return False
    return True


def matmul_nt(x: torch.Tensor, w: torch.Tensor, **kw) -> torch.Tensor:
    """``x[M,K] @ w[N,K]^T``."""
    if not _kernel_ok(x, w):
        y = x @ w.t()
        if kw.get("bias") is not None:
            y = y + kw["bias"]
        if kw.get("residual") is not None:
            y = y + kw["residual"]
        return y
    M, K = x.shape
    N = w.shape[0]
    return gemm_raw(x, False, w, False, M, N, K, **kw)


def matmul_nn(a: torch.Tensor, b: torch.Tensor, **kw) -> torch.Tensor:
    """``a[M,K] @ b[K,N]``."""
    if not _kernel_ok(a, b):
        return a @ b
    M, K = a.shape
    N = b.shape[1]
    return gemm_raw(a, False, b, True, M, N, K, **kw)


def matmul_tn(a: torch.Tensor, b: torch.Tensor, **kw) -> torch.Tensor:
    """``a[K,M]^T @ b[K,N]`` (the weight-gradient product ``dy^T x``)."""
    if not _kernel_ok(a, b):
        return a.t() @ b
    K, M = a.shape
    N = b.shape[1]
    return gemm_raw(a, True, b, True, M, N, K, **kw)


def matmul_tt(a: torch.Tensor, b: torch.Tensor, **kw) -> torch.Tensor:
    """``a[K,M]^T @ b[N,K]^T``."""
    if not _kernel_ok(a, b):
        return a.t() @ b.t()
    K, M = a.shape
    N = b.shape[0]
    return gemm_raw(a, True, b, False, M, N, K, **kw)


def _as_2d(x: torch.Tensor) -> torch.Tensor:
    x2 = x.reshape(-1, x.shape[-1])
    if x2.stride(-1) != 1:
        x2 = x2.contiguous()
    return x2


def _colsum(x2: torch.Tensor) -> torch.Tensor:
    """Sum over the rows of a 2-D tensor, fp32 accumulation, result in the input's dtype (the bias gradient)."""
    T, D = x2.shape
    if _kernel_ok(x2) and D % 8 == 0 and D <= 8192 and T > 0:
        lib = _lib.cuda_lib()
        out = torch.empty(D, dtype=x2.dtype, device=x2.device)
        scratch = torch.empty(lib.gf_norm_bwd_grid(T) * D, dtype=torch.float32, device=x2.device)
        _lib.check_rc(lib.gf_colsum_bf16(x2.data_ptr(), x2.stride(0), out.data_ptr(), scratch.data_ptr(), T, D, 0,
                                         _lib.stream_ptr()), "gf_colsum_bf16")
        return out
    return torch.sum(x2, 0, dtype=torch.float32).to(x2.dtype)   # fp32 accumulation without an fp32 copy of x


class _LinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, bias, residual):
        x2 = _as_2d(x)
        r2 = _as_2d(residual) if residual is not None else None
        y = matmul_nt(x2, w, bias=bias, residual=r2)
        ctx.save_for_backward(x2, w)
        ctx.has_bias = bias is not None
        ctx.has_res = residual is not None
        ctx.x_shape = x.shape
        return y.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, w = ctx.saved_tensors
        dy2 = _as_2d(dy)
        dx = dw = db = dres = None
        if ctx.needs_input_grad[0]:
            dx = matmul_nn(dy2, w).view(ctx.x_shape)
        if ctx.needs_input_grad[1]:
            dw = matmul_tn(dy2, x2)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = _colsum(dy2)
        if ctx.has_res and ctx.needs_input_grad[3]:
            dres = dy
        return dx, dw, db, dres


def linear(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None,
           residual: torch.Tensor | None = None) -> torch.Tensor:
    """``x @ w^T (+ bias) (+ residual)`` with the bias/residual adds fused into the GEMM epilogue."""
    if _kernel_ok(x, w):
        if not (torch.is_grad_enabled() and (x.requires_grad or w.requires_grad
                                             or (bias is not None and bias.requires_grad)
                                             or (residual is not None and residual.requires_grad))):
            # inference: straight to the kernel, no autograd node
            r2 = _as_2d(residual) if residual is not None else None
            x2 = _as_2d(x)
            y = gemm_raw(x2, False, w, False, x2.shape[0], w.shape[0], x2.shape[1], bias=bias, residual=r2)
            return y.view(*x.shape[:-1], w.shape[0])
        return _LinearFn.apply(x, w, bias, residual)
    y = torch.nn.functional.linear(x, w, bias)
    if residual is not None:
        y = y + residual
    return y


def matmul_fp32_split(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """``a @ b`` for fp32 CUDA matrices on the bf16 tensor-core kernel with close to fp32 accuracy.

    Each operand is split into two bf16 numbers (``x = hi + lo`` up to 2^-16 relative); the three significant cross
    terms ``hi hi + hi lo + lo hi`` are evaluated as ONE GEMM over a three times longer contraction
    (``[hi_a | hi_a | lo_a] @ [hi_b ; lo_b ; hi_b]``) with fp32 accumulation in tensor memory and an fp32 result.
    The relative error is about 2e-5 of ``|a| @ |b|``, between TF32 (1e-3) and an fp32 FMA loop (1e-6).
    Needs ``K`` and ``N`` to be multiples of 8 (16-byte rows for the copy engine)."""
    import ctypes

    M, K = a.shape
    K2, N = b.shape
    assert K == K2 and K % 8 == 0 and N % 8 == 0
    a = a if a.stride(1) == 1 else a.contiguous()
    b = b if b.stride(1) == 1 else b.contiguous()
    a3 = torch.empty(M, 3 * K, device=a.device, dtype=torch.bfloat16)
    b3 = torch.empty(3 * K, N, device=a.device, dtype=torch.bfloat16)
    lib = _lib.cuda_lib()
    L, I, P = ctypes.c_longlong, ctypes.c_int, ctypes.c_void_p
    lib.gf_split_bf16_cat.argtypes = [P, P, L, I, L, L, L, L, I, P]
    lib.gf_split_bf16_cat.restype = I
    _lib.check_rc(lib.gf_split_bf16_cat(a.data_ptr(), a3.data_ptr(), M, K, a.stride(0), 3 * K, K, 2 * K, 2,
                                        _lib.stream_ptr()), "gf_split_bf16_cat")
    _lib.check_rc(lib.gf_split_bf16_cat(b.data_ptr(), b3.data_ptr(), K, N, b.stride(0), N, K * N, 2 * K * N, 1,
                                        _lib.stream_ptr()), "gf_split_bf16_cat")
    return gemm_raw(a3, False, b3, True, M, N, 3 * K, out_dtype=torch.float32)


def _fp32_split_ok(a, b) -> bool:
    return (a.is_cuda and a.dtype == torch.float32 and b.dtype == torch.float32 and a.shape[1] % 8 == 0
            and b.shape[1] % 8 == 0 and a.shape[0] >= 64 and b.shape[1] >= 64 and a.shape[1] >= 16
            and not (torch.is_grad_enabled() and (a.requires_grad or b.requires_grad)))


def matmul(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """General matmul for the tensor API: 2-D bf16 CUDA operands use the tcgen05 kernel; 2-D fp32 CUDA operands
    use it through :func:`matmul_fp32_split`."""
    if a.dim() == 2 and b.dim() == 2 and _fp32_split_ok(a, b):
        return matmul_fp32_split(a, b)
    if a.dim() == 2 and b.dim() == 2 and _kernel_ok(a, b) and not (a.requires_grad or b.requires_grad):
        if a.stride(1) == 1 and b.stride(1) == 1:
            return matmul_nn(a, b)
        if a.stride(1) == 1 and b.stride(0) == 1:
            return matmul_nt(a, b.t())
    return torch.matmul(a, b)
