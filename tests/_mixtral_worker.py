"""Worker for the GPU Mixtral test: the expert-parallel engine (ZeRO-3 attention, experts sharded over the ranks) takes a
few optimizer steps; rank 0 saves the losses and some weights for the comparison with the fp32 CPU engine."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from ghost_flow_b200.models.configs import MixtralConfig  # noqa: E402
from ghost_flow_b200.ops import _lib  # noqa: E402
from ghost_flow_b200.parallel.mixtral import MixtralEngine  # noqa: E402
from ghost_flow_b200.parallel.symm import FusedComm  # noqa: E402
from ghost_flow_b200.parallel.zero3 import Comm, OptimConfig  # noqa: E402


def config():
    return MixtralConfig(vocab_size=2048, hidden_size=512, intermediate_size=1024, num_hidden_layers=2,
                         num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=512,
                         num_local_experts=8, num_experts_per_tok=2, router_aux_loss_coef=0.01)


def batch(world):
    g = torch.Generator().manual_seed(42)
    return torch.randint(0, 2048, (2 * world, 257), generator=g)


def main():
    kind, out_path, steps = sys.argv[1], sys.argv[2], int(sys.argv[3])
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    rank, world = dist.get_rank(), dist.get_world_size()
    cfg = config()
    comm = FusedComm(dev) if (kind == "fused" and world > 1) else Comm()
    eng = MixtralEngine(cfg, dev, tokens_per_rank=2 * 256, optim=OptimConfig(lr=5e-4, weight_decay=0.0), comm=comm,
                        seed=5, capacity_factor=float(world))
    tok = batch(world)[2 * rank:2 * rank + 2].to(dev)
    init = {k: v.cpu() for k, v in eng.state_dict(master=True).items() if ".moe." not in k}
    losses, aux = [], []
    for _ in range(steps):
        losses.append(float(eng.step(tok[:, :-1], tok[:, 1:])))
        aux.append(float(eng.last_stats["aux_loss"]))
    torch.cuda.synchronize()
    _lib.check_status(dev)
    wq = eng.gather_unit(eng.layers[1], master=True)["wqkv"].cpu()
    if rank == 0:
        e = eng.experts[1]
        torch.save({"losses": losses, "aux": aux, "wqkv": wq, "w13_e0": e.master["w13"][0].cpu(),
                    "w2_e0": e.master["w2"][0].cpu(), "gate": e.master["gate"].cpu(),
                    "fused": isinstance(comm, FusedComm), "init": init}, out_path)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
