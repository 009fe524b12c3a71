"""Bounded device waits: a wait that nothing satisfies ends by itself, reports through the status word, and leaves
the context usable."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_wait_on_flag_that_nobody_sets_returns_status_and_context_survives():
    from ghost_flow_b200.ops import _lib
    from ghost_flow_b200.ops.gemm import matmul_nt
    from ghost_flow_b200.parallel.fault import bounded_device_wait

    dev = torch.device("cuda", 0)
    pad = torch.zeros(64, dtype=torch.int32, device=dev)
    assert bounded_device_wait(pad, 0, 2, 1, limit=1 << 14) == 5          # timed out waiting for a peer flag
    pad[:2] = 1
    assert bounded_device_wait(pad, 0, 2, 1, limit=1 << 14) == 0          # flags present: returns at once
    a = torch.randn(256, 128, device=dev, dtype=torch.bfloat16)
    b = torch.randn(192, 128, device=dev, dtype=torch.bfloat16)
    y = matmul_nt(a, b)
    torch.cuda.synchronize()
    _lib.check_status(dev)
    assert torch.allclose(y.float(), a.float() @ b.float().t(), atol=0.5, rtol=2e-2)
