"""The allocation-free RMSNorm backward (``gf_rmsnorm_bwd_noalloc``), called through its exported C symbol
the way a host program without any tensor library would call it, against the regular entry point
(``gf_rmsnorm_bwd``, which takes a caller-provided scratch buffer).

The variant exists for callers that may not allocate device memory: plug-ins running inside another
framework's fixed memory plan, latency-critical loops that must never enter the allocator, plain C hosts.
Its scratch is a fixed array inside the library, shared by all calls on a device, so the test makes two
calls in a row with different sizes: the second must not be disturbed by what the first left behind.

This file sorts last on purpose, so a run that stops at the first failure has already run everything else.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel_err(a, b):
    a, b = a.float(), b.float()
    return ((a - b).norm() / (b.norm() + 1e-12)).item()


def _bind():
    from ghost_flow_b200.ops import _lib

    lib = ctypes.CDLL(str(_lib.lib_path()))
    P, I = ctypes.c_void_p, ctypes.c_int
    lib.gf_set_device.argtypes = [I]
    lib.gf_set_device.restype = None
    lib.gf_rmsnorm_bwd_noalloc.argtypes = [P, P, P, P, P, P, P, I, I, I, P]
    lib.gf_rmsnorm_bwd_noalloc.restype = I
    lib.gf_rmsnorm_bwd.argtypes = [P, P, P, P, P, P, P, P, I, I, I, P]
    lib.gf_rmsnorm_bwd.restype = I
    lib.gf_norm_bwd_grid.argtypes = [I]
    lib.gf_norm_bwd_grid.restype = I
    lib.gf_set_device(torch.cuda.current_device())
    return lib


def _case(lib, T, D, with_res, accumulate):
    dev = "cuda"
    x = torch.randn(T, D, device=dev, dtype=torch.bfloat16)
    w = (1 + 0.1 * torch.randn(D, device=dev)).to(torch.bfloat16)
    dy = torch.randn(T, D, device=dev, dtype=torch.bfloat16)
    dres = torch.randn(T, D, device=dev, dtype=torch.bfloat16) if with_res else None
    rstd = torch.rsqrt(x.float().pow(2).mean(-1) + 1e-6).contiguous()
    dw0 = torch.randn(D, device=dev).to(torch.bfloat16)
    stream = torch.cuda.current_stream().cuda_stream
    # regular entry point, scratch from the caller
    dx_ref = torch.empty_like(x)
    dw_ref = dw0.clone()
    scratch = torch.empty(lib.gf_norm_bwd_grid(T) * D, device=dev, dtype=torch.float32)
    rc = lib.gf_rmsnorm_bwd(x.data_ptr(), w.data_ptr(), dy.data_ptr(), rstd.data_ptr(),
                            dres.data_ptr() if with_res else None, dx_ref.data_ptr(), dw_ref.data_ptr(),
                            scratch.data_ptr(), T, D, accumulate, stream)
    assert rc == 0
    # allocation-free entry point: inputs and outputs only
    dx = torch.empty_like(x)
    dw = dw0.clone()
    rc = lib.gf_rmsnorm_bwd_noalloc(x.data_ptr(), w.data_ptr(), dy.data_ptr(), rstd.data_ptr(),
                                    dres.data_ptr() if with_res else None, dx.data_ptr(), dw.data_ptr(), T, D,
                                    accumulate, stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert _rel_err(dx, dx_ref) < 1e-2
    assert _rel_err(dw, dw_ref) < 1e-2
    # and both agree with fp32 PyTorch math
    xf, gf_, wf = x.float(), dy.float(), w.float()
    g = gf_ * wf
    r = rstd[:, None]
    dx_t = r * g - xf * r ** 3 * (g * xf).mean(-1, keepdim=True) + (dres.float() if with_res else 0)
    dw_t = (gf_ * xf * r).sum(0) + (dw0.float() if accumulate else 0)
    assert _rel_err(dx, dx_t) < 1e-2
    assert _rel_err(dw, dw_t) < 1e-2


def test_noalloc_matches_regular_entry_on_two_calls_in_a_row():
    lib = _bind()
    _case(lib, T=1000, D=4096, with_res=True, accumulate=0)   # fills all 148 scratch rows
    _case(lib, T=37, D=1024, with_res=False, accumulate=1)    # fewer, shorter rows right after: stale data ignored


def test_noalloc_at_its_documented_limits():
    """The longest row the built-in scratch takes (every thread works on its full set of vectors), and fewer
    rows than the scratch has partial-sum slots."""
    lib = _bind()
    _case(lib, T=300, D=8192, with_res=True, accumulate=0)
    _case(lib, T=5, D=8192, with_res=False, accumulate=1)
    _case(lib, T=147, D=256, with_res=True, accumulate=0)


def test_noalloc_refuses_misaligned_pointers_without_launching():
    """A sub-buffer that starts 2 bytes into an allocation cannot be read with 16-byte vectors: the call must come
    back with the bad-argument code and leave the outputs untouched (nothing ran on the device)."""
    lib = _bind()
    T, D = 16, 256
    base = torch.zeros(T * D + 8, device="cuda", dtype=torch.bfloat16)
    good = torch.zeros(T, D, device="cuda", dtype=torch.bfloat16)
    rstd = torch.ones(T + 1, device="cuda", dtype=torch.float32)
    dx = torch.full((T, D), 7.0, device="cuda", dtype=torch.bfloat16)
    dw = torch.full((D,), 7.0, device="cuda", dtype=torch.bfloat16)
    st = torch.cuda.current_stream().cuda_stream
    off = base.data_ptr() + 2                                   # 2-byte aligned only
    for args in ((off, good.data_ptr(), good.data_ptr(), rstd.data_ptr(), None),      # x misaligned
                 (good.data_ptr(), good.data_ptr(), off, rstd.data_ptr(), None),      # dy misaligned
                 (good.data_ptr(), good.data_ptr(), good.data_ptr(), rstd.data_ptr() + 2, None),   # rstd misaligned
                 (good.data_ptr(), good.data_ptr(), good.data_ptr(), rstd.data_ptr(), off)):       # dres misaligned
        rc = lib.gf_rmsnorm_bwd_noalloc(args[0], args[1], args[2], args[3], args[4], dx.data_ptr(), dw.data_ptr(),
                                        T, D, 0, st)
        assert rc == -1
    assert lib.gf_rmsnorm_bwd_noalloc(good.data_ptr(), good.data_ptr(), good.data_ptr(), rstd.data_ptr(), None,
                                      dx.data_ptr() + 2, dw.data_ptr(), T, D, 0, st) == -1
    assert lib.gf_rmsnorm_bwd_noalloc(good.data_ptr(), None, good.data_ptr(), rstd.data_ptr(), None,
                                      dx.data_ptr(), dw.data_ptr(), T, D, 0, st) == -1
    torch.cuda.synchronize()
    assert bool((dx == 7).all()) and bool((dw == 7).all())


def test_noalloc_rejects_rows_longer_than_its_scratch(capfd):
    lib = _bind()
    t = torch.zeros(8, device="cuda", dtype=torch.bfloat16)
    rc = lib.gf_rmsnorm_bwd_noalloc(t.data_ptr(), t.data_ptr(), t.data_ptr(), t.data_ptr(), None, t.data_ptr(),
                                    t.data_ptr(), 4, 8192 + 8, 0, torch.cuda.current_stream().cuda_stream)
    assert rc == -4
    assert "exceeds the built-in scratch" in capfd.readouterr().err
