"""ctypes binding of ``libgfb200.so`` (the sm_100a kernels) and ``libghostflow.so`` (host C++).

The CUDA library is mandatory on a machine with a GPU: :func:`cuda_lib` raises instead of
silently falling back, so a missing or stale build can never hide behind PyTorch ops.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_longlong, c_void_p
from pathlib import Path

import torch

_PKG = Path(__file__).resolve().parent.parent
_CUDA_LIB = None
_HOST_LIB = None

P = c_void_p
I = c_int
L = c_longlong
F = c_float

# name -> argtypes (restype is always int unless listed in _RESTYPES)
_SIGS = {
    "gf_sm_count": [],
    "gf_device_count": [],
    "gf_version": [],
    "gf_set_device": [I],
    "gf_gemm_bf16": [P, P, P, I, I, I, I, L, I, L, L, I, I, P, P, L, F, P, I, I, P, I, I, P],
    "gf_norm_bwd_grid": [I],
    "gf_rmsnorm_fwd": [P, P, P, P, P, P, I, I, F, P],
    "gf_rmsnorm_bwd": [P, P, P, P, P, P, P, P, I, I, I, P],
    "gf_layernorm_fwd": [P, P, P, P, P, P, I, I, F, P],
    "gf_layernorm_bwd": [P, P, P, P, P, P, P, P, P, I, I, I, P],
    "gf_rope": [P, P, P, I, I, I, L, L, I, I, I, I, P],
    "gf_swiglu_fwd": [P, P, L, I, P],
    "gf_scale_by_dev_scalar": [P, L, P, P],
    "gf_swiglu_bwd": [P, P, P, L, I, P],
    "gf_unary_fwd": [P, P, L, I, I, P],
    "gf_unary_bwd_bf16": [P, P, P, L, I, P],
    "gf_op_chain": [P, P, L, P, I, I, P],
    "gf_binary": [P, P, P, L, I, F, I, P],
    "gf_reduce": [P, P, P, L, I, I, P],
    "gf_softmax_rows": [P, P, I, I, I, I, P],
    "gf_xent_fused": [P, P, P, P, I, I, L, F, L, P],
    "gf_adam_flat": [P, P, P, P, P, L, F, F, F, F, F, I, F, I, I, P, P],
    "gf_adam_flat_dev": [P, P, P, P, P, L, F, F, F, F, F, I, F, I, I, P, P, P],
    "gf_counter_add": [P, I, P],
    "gf_colsum_bf16": [P, L, P, P, I, I, I, P],
    "gf_sgd_flat": [P, P, P, P, L, F, F, F, F, I, I, F, I, P],
    "gf_grad_sumsq": [P, L, P, I, P],
    "gf_flash_attn_fwd": [P, P, P, P, P, I, I, I, I, I, L, L, L, L, F, I, P, P],
    "gf_flash_attn_fwd2": [P, P, P, P, P, I, I, I, I, I, L, L, L, L, F, I, P, P],
    "gf_flash_attn_fwd3": [P, P, P, P, P, I, I, I, I, I, L, L, L, L, F, I, P, P],
    "gf_attn_decode": [P, L, P, P, I, P, I, P, L, I, I, I, I, F, I, P, P],
    "gf_flash_attn_bwd": [P, P, P, P, P, P, P, P, P, I, I, I, I, I, L, L, L, L, L, L, F, I, P, P],
    "gf_attn_bwd_prep": [P, P, P, P, I, I, I, I, L, L, P],
    "gf_flash_attn_bwd2": [P, P, P, P, P, P, P, P, P, I, I, I, I, I, L, L, L, L, L, L, F, I, P, P],
    "gf_attn_bwd_prep2": [P, P, P, P, P, P, I, I, I, I, L, L, P],
    "gf_dq_tiles_to_bf16": [P, P, I, I, I, I, L, F, P],
    "gf_cast_f32_to_bf16_2d": [P, P, L, I, L, L, F, P],
}


def _bind(lib, sigs):
    for name, args in sigs.items():
        try:
            fn = getattr(lib, name)
        except AttributeError:
            continue
        fn.argtypes = args
        fn.restype = c_int
    return lib


CHECKED = os.environ.get("GF_CHECKED", "0") == "1"


def lib_path() -> Path:
    """The kernel library; ``GF_CHECKED=1`` selects the build whose data-dependent indices are range-checked."""
    return _PKG / "lib" / ("libgfb200_checked.so" if CHECKED else "libgfb200.so")


def host_lib_path() -> Path:
    return _PKG / "lib" / "libghostflow.so"


def cuda_lib():
    """Returns the loaded CUDA kernel library; builds it first if the .so is missing."""
    global _CUDA_LIB
    if _CUDA_LIB is None:
        path = lib_path()
        if not path.exists():
            from ..csrc.build import build

            build()
        if not path.exists():
            raise RuntimeError(
                f"{path} is missing: run `python -m ghost_flow_b200.csrc.build` (needs nvcc). "
                "CUDA tensors are never routed to a fallback."
            )
        _CUDA_LIB = _bind(ctypes.CDLL(str(path), mode=ctypes.RTLD_GLOBAL), _SIGS)
    return _CUDA_LIB


def launch_count() -> int:
    """Kernels launched by the library so far in this process."""
    fn = cuda_lib().gf_launch_count
    fn.restype = ctypes.c_longlong
    fn.argtypes = []
    return int(fn())


def has_cuda_lib() -> bool:
    return lib_path().exists()


def host_lib():
    """Returns the host-only C++ library (checkpoint formats, C ABI, CPU reference math)."""
    global _HOST_LIB
    if _HOST_LIB is None:
        path = host_lib_path()
        if not path.exists():
            from ..csrc.build import build

            build()
        _HOST_LIB = ctypes.CDLL(str(path))
    return _HOST_LIB


_BOUND_DEVICE = -1


def stream_ptr() -> int:
    """Current CUDA stream handle; also keeps the kernel library's device in step with PyTorch's
    (the library carries its own copy of the CUDA runtime, with its own current-device state)."""
    global _BOUND_DEVICE
    dev = torch.cuda.current_device()
    if dev != _BOUND_DEVICE:
        cuda_lib().gf_set_device(dev)
        _BOUND_DEVICE = dev
    return torch.cuda.current_stream().cuda_stream


_STATUS = {}


def status_word(device=None) -> torch.Tensor:
    """Per-device int32 word that kernels write a bounded-wait error code into (0 = ok)."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    key = dev.index if dev.index is not None else torch.cuda.current_device()
    t = _STATUS.get(key)
    if t is None:
        # word 0: error code; words 1..7: {site, block, thread, index lo/hi, limit lo/hi} of a checked build's report
        t = torch.zeros(8, dtype=torch.int32, device=dev)
        _STATUS[key] = t
        lib = cuda_lib()
        if hasattr(lib, "gf_set_check_buffer"):
            lib.gf_set_check_buffer.argtypes = [c_int, c_void_p]
            lib.gf_set_check_buffer(key, t.data_ptr())
    return t


_ERR_NAMES = {
    1: "consumer timed out waiting for a TMA stage",
    2: "producer timed out waiting for a free stage",
    3: "epilogue timed out waiting for the accumulator",
    4: "MMA issuer timed out waiting for a drained accumulator",
    5: "timed out waiting for a peer flag",
    6: "timed out in the softmax hand-off",
    7: "bad argument seen on the device",
    8: "more rows were routed to a rank than its buffers hold",
    9: "index out of range (checked build)",
}
_SITES = {1: "moe_dispatch_kernel: expert id", 2: "moe_dispatch_kernel: destination row",
          3: "grouped GEMM scatter epilogue: rank of a return address", 4: "moe_combine_kernel: slot row"}


class KernelStatusError(RuntimeError):
    pass


def check_status(device=None, reset: bool = True) -> None:
    """Synchronises and raises if any kernel since the last check recorded an error code, or if a guard block behind
    a carve-out of an arena / workspace was overwritten (``parallel.canary``)."""
    w = status_word(device)
    rec = w.tolist()
    code = rec[0]
    if code != 0:
        if reset:
            w.zero_()
        detail = ""
        if code == 9:
            index = (rec[5] << 32) | (rec[4] & 0xFFFFFFFF)
            limit = (rec[7] << 32) | (rec[6] & 0xFFFFFFFF)
            detail = (f" at {_SITES.get(rec[1], f'site {rec[1]}')}, block {rec[2]}, thread {rec[3]}: index {index} "
                      f"outside [0, {limit}); the access was skipped")
        raise KernelStatusError(f"ghost_flow_b200 kernel status {code}: {_ERR_NAMES.get(code, 'unknown')}{detail}")
    import sys

    canary = sys.modules.get("ghost_flow_b200.parallel.canary")     # only if something planted guard blocks
    if canary is not None:
        canary.check_all()


def check_rc(rc: int, what: str) -> None:
    if rc != 0:
        names = {-1: "bad argument", -2: "CUDA launch error", -3: "tensor-map encode failed", -4: "size too large"}
        extra = ""
        if rc == -2:
            extra = f" ({torch.cuda.is_available() and 'see cudaGetLastError' or 'no GPU'})"
        raise RuntimeError(f"{what} failed: {names.get(rc, rc)}{extra}")


DEBUG_SYNC = os.environ.get("GF_DEBUG_SYNC", "0") == "1"


def flash_fwd_fn():
    """Forward attention launcher: the kernel that keeps P in tensor memory, unless GF_FA_FWD=2 selects the
    earlier two-tile kernel (P through shared memory) or GF_FA_FWD=1 the single-tile one."""
    lib = cuda_lib()
    which = os.environ.get("GF_FA_FWD", "3")
    if which == "1":
        return lib.gf_flash_attn_fwd
    if which == "2":
        return lib.gf_flash_attn_fwd2
    return lib.gf_flash_attn_fwd3


def flash_attn_backward(q, k, v, o, do, lse, dq, dk, dv, B, S, Hq, Hkv, D, ld, scale, causal) -> None:
    """Launches the attention backward (statistics kernel, main kernel, fp32 -> bf16 conversion of dQ) on the
    current stream. All tensors are bf16 CUDA tensors or views; ``ld`` maps ``q k v o do dq dk dv`` to their row
    pitch in elements. ``GF_FA_BWD=1`` selects the first-generation kernel (compute warps also drain dQ)."""
    lib = cuda_lib()
    st = stream_ptr()
    dev = q.device
    status = status_word(dev).data_ptr()
    delta = torch.empty((B, Hq, S), dtype=torch.float32, device=dev)
    dq_acc = torch.empty((B * S, Hq * D), dtype=torch.float32, device=dev)
    c = 1 if causal else 0
    if os.environ.get("GF_FA_BWD", "2") == "1":
        check_rc(lib.gf_attn_bwd_prep(o.data_ptr(), do.data_ptr(), delta.data_ptr(), dq_acc.data_ptr(), B, S, Hq, D,
                                      ld["o"], ld["do"], st), "gf_attn_bwd_prep")
        check_rc(lib.gf_flash_attn_bwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), do.data_ptr(), lse.data_ptr(),
                                       delta.data_ptr(), dq_acc.data_ptr(), dk.data_ptr(), dv.data_ptr(), B, S, Hq,
                                       Hkv, D, ld["q"], ld["k"], ld["v"], ld["do"], ld["dk"], ld["dv"], float(scale),
                                       c, status, st), "gf_flash_attn_bwd")
        check_rc(lib.gf_cast_f32_to_bf16_2d(dq_acc.data_ptr(), dq.data_ptr(), B * S, Hq * D, Hq * D, ld["dq"], 1.0,
                                            st), "gf_cast_f32_to_bf16_2d")
    else:
        nlse2 = torch.empty((B, Hq, S), dtype=torch.float32, device=dev)
        check_rc(lib.gf_attn_bwd_prep2(o.data_ptr(), do.data_ptr(), lse.data_ptr(), delta.data_ptr(),
                                       nlse2.data_ptr(), dq_acc.data_ptr(), B, S, Hq, D, ld["o"], ld["do"], st),
                 "gf_attn_bwd_prep2")
        check_rc(lib.gf_flash_attn_bwd2(q.data_ptr(), k.data_ptr(), v.data_ptr(), do.data_ptr(), nlse2.data_ptr(),
                                        delta.data_ptr(), dq_acc.data_ptr(), dk.data_ptr(), dv.data_ptr(), B, S, Hq,
                                        Hkv, D, ld["q"], ld["k"], ld["v"], ld["do"], ld["dk"], ld["dv"],
                                        float(scale), c, status, st), "gf_flash_attn_bwd2")
        # the main kernel leaves dQ / scale in the accumulator, tile by tile ([B, Hq, S / 64, 64, D])
        check_rc(lib.gf_dq_tiles_to_bf16(dq_acc.data_ptr(), dq.data_ptr(), B, S, Hq, D, ld["dq"], float(scale), st),
                 "gf_dq_tiles_to_bf16")
