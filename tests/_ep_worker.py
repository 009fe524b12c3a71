"""Worker for the expert-parallel MoE test (one rank per GPU, launched with torch.distributed.run)."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from ghost_flow_b200.ops import _lib  # noqa: E402
from ghost_flow_b200.parallel.ep import ExpertParallelMoE  # noqa: E402


def rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


def main():
    out_path = sys.argv[1]
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    rank, world = dist.get_rank(), dist.get_world_size()
    res = {}
    for (T, d, f, E, k) in [(512, 256, 384, 8, 2), (1024, 512, 512, 4 * world, 2)]:
        moe = ExpertParallelMoE(d, f, E, k, T, dev, seed=11)
        g = torch.Generator(device="cpu").manual_seed(5)
        moe.gate_pad[:E] = (torch.randn(E, d, generator=g) * 0.5).to(torch.bfloat16).to(dev)
        torch.manual_seed(100 + rank)
        for it in range(2):                         # second pass reuses buffers and flags with a later epoch
            x = torch.randn(T, d, device=dev, dtype=torch.bfloat16)
            dy = torch.randn(T, d, device=dev, dtype=torch.bfloat16) * 0.1
            for v in moe.grads.values():
                v.zero_()
            y, ctx = moe.forward(x)
            dx = moe.backward(ctx, dy)
            torch.cuda.synchronize()
            _lib.check_status(dev)
            w13f, w2f = moe.full_weights()
            xr = x.float().requires_grad_(True)
            gate = moe.gate.float().requires_grad_(True)
            w13 = w13f.float().requires_grad_(True)
            w2 = w2f.float().requires_grad_(True)
            saved, moe.gate = moe.gate, gate
            ref = moe.dense_reference(xr, w13, w2)
            moe.gate = saved
            ref.backward(dy.float())
            g13, g2 = w13.grad.clone(), w2.grad.clone()
            dist.all_reduce(g13)
            dist.all_reduce(g2)
            lo, hi = rank * moe.el, (rank + 1) * moe.el
            tag = f"T{T}_E{E}_it{it}"
            res[f"y_{tag}"] = rel(y, ref)
            res[f"dx_{tag}"] = rel(dx, xr.grad)
            res[f"dw13_{tag}"] = rel(moe.grads["w13"], g13[lo:hi])
            res[f"dw2_{tag}"] = rel(moe.grads["w2"], g2[lo:hi])
            res[f"dgate_{tag}"] = rel(moe.grads["gate"], gate.grad)
            res[f"counts_{tag}"] = 0.0 if int(moe.expert_counts().sum()) == T * k else 1.0
    worst = torch.tensor([max(res.values())], device=dev)
    dist.all_reduce(worst, op=dist.ReduceOp.MAX)
    res["worst_over_ranks"] = float(worst)
    if rank == 0:
        torch.save(res, out_path)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
