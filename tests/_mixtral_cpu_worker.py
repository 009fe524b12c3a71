"""gloo worker: the Mixtral engine on CPU ranks (ZeRO-3 attention units, experts split over the ranks, router gradient
all-reduced); rank 0 writes the loss curve and some weights."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from ghost_flow_b200.models.configs import MixtralConfig  # noqa: E402
from ghost_flow_b200.parallel.mixtral import MixtralEngine  # noqa: E402
from ghost_flow_b200.parallel.zero3 import Comm, OptimConfig  # noqa: E402


def config(aux):
    return MixtralConfig(vocab_size=128, hidden_size=32, intermediate_size=64, num_hidden_layers=2,
                         num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=32,
                         num_local_experts=4, num_experts_per_tok=2, router_aux_loss_coef=aux)


def batch():
    g = torch.Generator().manual_seed(11)
    return torch.randint(0, 128, (4, 17), generator=g)


def run(world, rank, aux, steps=4):
    cfg = config(aux)
    tok = batch()
    per = tok.shape[0] // world
    mine = tok[rank * per:(rank + 1) * per]
    eng = MixtralEngine(cfg, "cpu", tokens_per_rank=per * 16, optim=OptimConfig(lr=3e-3, weight_decay=0.0),
                        dtype=torch.float32, seed=3, comm=Comm() if world > 1 else None)
    losses = [float(eng.step(mine[:, :-1], mine[:, 1:])) for _ in range(steps)]
    sd = eng.state_dict()
    return {"losses": losses, "w13": sd["layers.1.moe.w13"], "gate": sd["layers.0.moe.gate"],
            "wqkv": sd["layers.1.wqkv"]}


def main():
    out, aux = sys.argv[1], float(sys.argv[2])
    dist.init_process_group("gloo")
    res = run(dist.get_world_size(), dist.get_rank(), aux)
    if dist.get_rank() == 0:
        torch.save(res, out)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
