"""Worker for the multi-GPU ZeRO-2 test (one rank per GPU): trains a small GPT with the generic ZeRoOptimizer on the
requested collective path and writes rank 0's loss curve and one parameter."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from ghost_flow_b200.models.configs import GPTConfig  # noqa: E402
from ghost_flow_b200.models.gpt import GPTForCausalLM  # noqa: E402
from ghost_flow_b200.ops import _lib  # noqa: E402
from ghost_flow_b200.parallel.distributed import ZeRoConfig, ZeRoOptimizer, ZeRoStage  # noqa: E402


def main():
    kind, out, steps = sys.argv[1], sys.argv[2], int(sys.argv[3])
    # kind: fused | nccl, optionally followed by _graph (whole step replayed from a CUDA graph) and / or _late
    # (collectives after backward instead of from gradient hooks)
    graph, late = "_graph" in kind, "_late" in kind
    kind = kind.split("_")[0]
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    rank, world = dist.get_rank(), dist.get_world_size()
    cfg = GPTConfig(vocab_size=512, n_positions=128, n_embd=128, n_layer=2, n_head=4, n_inner=512)
    cfg.dropout = 0.0
    torch.manual_seed(0)
    model = GPTForCausalLM(cfg).to(dev, torch.bfloat16)
    # small buckets so that several of them are in flight
    opt = ZeRoOptimizer(model.parameters(), ZeRoConfig(stage=ZeRoStage.Stage2, world_size=world, rank=rank, lr=1e-3,
                                                       betas=(0.9, 0.95), weight_decay=0.1, bucket_size=150_000),
                        comm=kind, overlap=not late, capturable=graph)
    g = torch.Generator().manual_seed(7)
    ids = torch.randint(0, cfg.vocab_size, (world * 2, 129), generator=g)
    mine = ids[rank * 2:(rank + 1) * 2].to(dev)
    losses = []

    def train(x, y):
        opt.zero_grad()
        res = model(x, labels=y)
        loss = res[0] if isinstance(res, tuple) else res
        loss.backward()
        opt.step()
        return loss.detach()

    x, y = mine[:, :-1].contiguous(), mine[:, 1:].contiguous()
    if graph:
        from ghost_flow_b200.utils import GraphedStep

        gs = GraphedStep(train, (x, y), warmup=2)        # two real steps, then every further one is a replay
        losses = [float(l) for l in gs.warmup_outputs]
        for _ in range(steps - 2):
            losses.append(float(gs(x, y)))
    else:
        for _ in range(steps):
            losses.append(float(train(x, y)))
    torch.cuda.synchronize()
    _lib.check_status(dev)
    w = [p for p in model.parameters()][-3].detach().float().cpu()
    if rank == 0:
        torch.save({"losses": losses, "w": w, "buckets": len(opt.buckets), "fused": opt._fc is not None,
                    "overlap": opt.overlap, "graph": graph}, out)
    if graph:
        gs.release()
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
