"""Worker for the fused tensor-parallel kernel tests (one rank per GPU, launched with torch.distributed.run)."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from ghost_flow_b200.ops import _lib  # noqa: E402
from ghost_flow_b200.parallel.tp import AllGatherGemm, GemmReduceScatter  # noqa: E402


def rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


def timed(fn, iters=10):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / iters], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t)


def main():
    out_path = sys.argv[1]
    big = len(sys.argv) > 2 and sys.argv[2] == "big"
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    rank, world = dist.get_rank(), dist.get_world_size()
    torch.manual_seed(100 + rank)
    res = {}
    shapes = [(512, 256, 384), (1024, 1024, 768)] + ([(16384, 8192, 3584)] if big else [])
    for (T, K, N) in shapes:
        ag = AllGatherGemm(T, K, dev)
        x = torch.randn(T // world, K, device=dev, dtype=torch.bfloat16)
        w = torch.randn(N, K, device=dev, dtype=torch.bfloat16) * 0.05
        for it in range(3):                      # repeated calls exercise the parity double-buffering
            x = x + 0.01 * it
            got, ref = ag(x, w), ag.reference(x, w)
            res[f"ag_gemm_{T}x{K}x{N}_{it}"] = rel(got, ref)
        if big:
            res[f"ag_gemm_{T}x{K}x{N}_ms_fused"] = timed(lambda: ag(x, w))
            res[f"ag_gemm_{T}x{K}x{N}_ms_nccl"] = timed(lambda: ag.reference(x, w))
        rs = GemmReduceScatter(T, N, dev)
        xl = torch.randn(T, K // world if K % world == 0 else K, device=dev, dtype=torch.bfloat16)
        wl = torch.randn(N, xl.shape[1], device=dev, dtype=torch.bfloat16) * 0.05
        resid = torch.randn(T // world, N, device=dev, dtype=torch.bfloat16)
        for it in range(3):
            xl = xl + 0.01 * it
            got, ref = rs(xl, wl, residual=resid), rs.reference(xl, wl, residual=resid)
            res[f"gemm_rs_{T}x{K}x{N}_{it}"] = rel(got, ref)
        if big:
            res[f"gemm_rs_{T}x{K}x{N}_ms_fused"] = timed(lambda: rs(xl, wl))
            res[f"gemm_rs_{T}x{K}x{N}_ms_nccl"] = timed(lambda: rs.reference(xl, wl))
    torch.cuda.synchronize()
    _lib.check_status(dev)
    if rank == 0:
        torch.save(res, out_path)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
