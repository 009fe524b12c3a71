"""Worker for the GPU context-parallel test (ring attention and Ulysses over NCCL, kernels on the GPU)."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from ghost_flow_b200.ops import _lib, raw  # noqa: E402
from ghost_flow_b200.parallel.context import (ContextParallelAttention, UlyssesAttention,  # noqa: E402
                                               ZigZagContextParallelAttention, zigzag_rows)


def rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


def main():
    out_path = sys.argv[1]
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    rank, world = dist.get_rank(), dist.get_world_size()
    B, S, H, Hkv, D = 1, 512, 8, 4, 128
    g = torch.Generator(device="cpu").manual_seed(3)
    mk = lambda c: torch.randn(B * S * world, c, generator=g).to(torch.bfloat16).to(dev)  # noqa: E731
    q, k, v, do = mk(H * D), mk(Hkv * D), mk(Hkv * D), mk(H * D)
    o_ref, lse_ref = raw.attn_fwd(q, k, v, B, S * world, H, Hkv, D, True)
    dq_r, dk_r, dv_r = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    raw.attn_bwd(q, k, v, o_ref, do, lse_ref, dq_r, dk_r, dv_r, B, S * world, H, Hkv, D, True)
    sl = slice(rank * S, (rank + 1) * S)
    ql, kl, vl, dol = (t[sl].contiguous() for t in (q, k, v, do))
    res = {}
    cp = ContextParallelAttention(B, S, H, Hkv, D, causal=True)
    o, lse = cp.forward(ql, kl, vl)
    dq, dk, dv = cp.backward(ql, kl, vl, o, lse, dol)
    res.update(ring_o=rel(o, o_ref[sl]), ring_dq=rel(dq, dq_r[sl]), ring_dk=rel(dk, dk_r[sl]), ring_dv=rel(dv, dv_r[sl]))
    ul = UlyssesAttention(B, S, H, Hkv, D, causal=True)
    o2, ctx = ul.forward(ql, kl, vl)
    dq2, dk2, dv2 = ul.backward(ctx, dol)
    res.update(ulysses_o=rel(o2, o_ref[sl]), ulysses_dq=rel(dq2, dq_r[sl]), ulysses_dk=rel(dk2, dk_r[sl]),
               ulysses_dv=rel(dv2, dv_r[sl]))
    # load-balanced (zig-zag) assignment; with 512 local rows the halves are 256-row blocks, a size both
    # attention kernels take
    rows = zigzag_rows(S * world, world, rank).to(dev)
    qz, kz, vz, doz = (t[rows].contiguous() for t in (q, k, v, do))
    zz = ZigZagContextParallelAttention(B, S, H, Hkv, D)
    oz, lz = zz.forward(qz, kz, vz)
    dqz, dkz, dvz = zz.backward(qz, kz, vz, oz, lz, doz)
    res.update(zigzag_o=rel(oz, o_ref[rows]), zigzag_dq=rel(dqz, dq_r[rows]), zigzag_dk=rel(dkz, dk_r[rows]),
               zigzag_dv=rel(dvz, dv_r[rows]))
    torch.cuda.synchronize()
    _lib.check_status(dev)
    worst = torch.tensor([max(res.values())], device=dev)
    dist.all_reduce(worst, op=dist.ReduceOp.MAX)
    res["worst_over_ranks"] = float(worst)
    if rank == 0:
        torch.save(res, out_path)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
