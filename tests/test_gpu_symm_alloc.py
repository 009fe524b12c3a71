"""The library's own allocator against the real driver, one rank: create, reserve, map, set access, use the memory
from torch and from one of this library's kernels, unmap and release. (The multi-process descriptor exchange is
covered on the host stand-in, tests/test_symm_alloc_cpu.py.)

The allocator had only run against its host stand-in when this test was written, so the check runs in a child
process (a wrong call into the driver must not take the test session down) and is marked as allowed to fail: it
reports XPASS where the driver path works and XFAIL with the child's output where it does not."""
import os
import subprocess
import sys
import textwrap

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CHILD = textwrap.dedent("""
    import sys, torch
    sys.path.insert(0, {root!r})
    from ghost_flow_b200 import ops
    from ghost_flow_b200.parallel.symm_alloc import SymmetricAllocation
    try:
        a = SymmetricAllocation(1 << 20, 0, 1, device=torch.cuda.current_device())
    except RuntimeError as e:
        print("refused:", e)
        sys.exit(77)
    assert a.bytes_per_rank >= (1 << 20) and a.ptrs[0] % 256 == 0
    t = a.tensor(dtype=torch.int32)
    assert t.is_cuda and t.data_ptr() == a.ptrs[0]
    t.fill_(7)
    t[:4] = torch.tensor([1, 2, 3, 4], dtype=torch.int32, device=t.device)
    assert t[:6].cpu().tolist() == [1, 2, 3, 4, 7, 7] and int(t.sum().item()) == 7 * (t.numel() - 4) + 10
    x = a.tensor(dtype=torch.bfloat16)[:4096]
    x.copy_(torch.linspace(-2, 2, 4096, device=x.device).to(torch.bfloat16))
    y = ops.unary(x, "relu")                       # one of the library's kernels reading the mapped memory
    assert torch.equal(y, torch.relu(x))
    torch.cuda.synchronize()
    del t, x
    a.close()
    print("ok")
""")


@pytest.mark.xfail(strict=False, reason="first contact of the allocator with a real driver")
def test_own_allocation_is_usable_device_memory():
    r = subprocess.run([sys.executable, "-c", CHILD.format(root=ROOT)], capture_output=True, text=True, timeout=300)
    if r.returncode == 77:
        pytest.skip("the driver refused the allocation: " + r.stdout.strip()[-300:])
    assert r.returncode == 0 and r.stdout.strip().endswith("ok"), (r.returncode, r.stdout[-500:], r.stderr[-1500:])
