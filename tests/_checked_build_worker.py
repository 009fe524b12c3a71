"""Runs under GF_CHECKED=1: the checked kernel library on a healthy MoE layer (no report) and on a routing table with
one corrupted expert id (the dispatch kernel skips that row and reports where and what)."""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from ghost_flow_b200.ops import _lib  # noqa: E402
from ghost_flow_b200.parallel import ep  # noqa: E402


def main():
    lib = _lib.cuda_lib()
    assert _lib.CHECKED and lib.gf_checked_build() == 1, "the checked library was not loaded"
    dev = torch.device("cuda", 0)
    T, d, f, E, k = 256, 256, 512, 8, 2
    moe = ep.ExpertParallelMoE(d, f, E, k, T, dev, seed=1)
    x = (0.5 * torch.randn(T, d, device=dev)).to(torch.bfloat16)
    y, ctx = moe.forward(x)
    ref = moe.dense_reference(x)
    torch.cuda.synchronize()
    _lib.check_status(dev)                                   # healthy run: no report, guard blocks intact
    rel = ((y.float() - ref).norm() / ref.norm()).item()
    assert rel < 3e-2, rel
    # one corrupted entry of the routing table, replayed through the backward-style dispatch (rows are reused)
    bad = ctx.idx.clone()
    bad[3, 1] = E + 5
    dy = torch.randn(T, d, device=dev, dtype=torch.bfloat16)
    mlib = ep._bind()
    moe.epoch += 1
    _lib.check_rc(mlib.gf_moe_dispatch(dy.data_ptr(), dy.stride(0), bad.data_ptr(), ctx.w.data_ptr(), T, k, d, E, 1, 0,
                                       moe.rows_cap, moe.send_base.data_ptr(), moe.cursor.data_ptr(),
                                       ctx.dest_row.data_ptr(), 1, moe.p["dys"], moe.p["ret"], moe.p["flags"],
                                       ep.FLAG_DISPATCH, moe.epoch, moe.done.data_ptr(), _lib.stream_ptr()),
                  "gf_moe_dispatch")
    torch.cuda.synchronize()
    try:
        _lib.check_status(dev)
    except _lib.KernelStatusError as e:
        msg = str(e)
        assert "expert id" in msg and f"index {E + 5} outside [0, {E})" in msg, msg
        print("REPORT:", msg)
    else:
        raise AssertionError("the corrupted expert id was not reported")
    # the context is intact and the layer still works
    y2, _ = moe.forward(x)
    torch.cuda.synchronize()
    _lib.check_status(dev)
    assert torch.equal(y, y2)
    print("OK")


if __name__ == "__main__":
    main()
