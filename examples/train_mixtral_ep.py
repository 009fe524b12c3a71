"""Mixtral-style mixture-of-experts training with expert parallelism = world size.

    python examples/train_mixtral_ep.py                                            # one process, CPU or one GPU
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \
        --master-port 29570 examples/train_mixtral_ep.py                            # experts split over the ranks

Attention and norm parameters are ZeRO-3 units (sharded over the ranks, gathered per layer, gradients reduce-scattered
into AdamW); each rank owns ``experts / world`` SwiGLU experts per layer with their optimizer state; tokens travel to
their experts and back (peer-memory kernels on GPUs, gloo collectives on CPU ranks); the load-balancing loss is part
of the gradient. The reference's mixture of experts is a single-process CPU loop
(ghostflow-nn/src/mixture_of_experts.rs:212-274).
"""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from ghost_flow_b200.models.configs import MixtralConfig  # noqa: E402
from ghost_flow_b200.parallel.mixtral import MixtralEngine  # noqa: E402
from ghost_flow_b200.parallel.zero3 import Comm, OptimConfig  # noqa: E402


def main():
    world = int(os.environ.get("WORLD_SIZE", 1))
    cuda = torch.cuda.is_available()
    local = int(os.environ.get("LOCAL_RANK", 0))
    dev = torch.device("cuda", local) if cuda else torch.device("cpu")
    if cuda:
        torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl" if cuda else "gloo", **({"device_id": dev} if cuda else {}))
    rank = dist.get_rank() if world > 1 else 0
    d = 512 if cuda else 64                      # head_dim 128 on the GPU kernels
    cfg = MixtralConfig(vocab_size=1024, hidden_size=d, intermediate_size=2 * d, num_hidden_layers=2,
                        num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=256,
                        num_local_experts=4, num_experts_per_tok=2, router_aux_loss_coef=0.01)
    seq, micro = (256, 2) if cuda else (32, 2)
    comm = None
    if world > 1:
        if cuda:
            from ghost_flow_b200.parallel.symm import FusedComm
            comm = FusedComm(dev)
        else:
            comm = Comm()
    eng = MixtralEngine(cfg, dev, tokens_per_rank=micro * seq, optim=OptimConfig(lr=2e-3, weight_decay=0.0),
                        dtype=torch.bfloat16 if cuda else torch.float32, comm=comm, seed=0)
    g = torch.Generator().manual_seed(1 + rank)
    ids = torch.randint(0, cfg.vocab_size, (micro, seq + 1), generator=g).to(dev)     # one fixed batch: the loss must fall
    for step in range(8):
        loss = eng.step(ids[:, :-1], ids[:, 1:])
        if rank == 0:
            print(f"step {step}  loss {float(loss):.4f}  aux {float(eng.last_stats['aux_loss']):.4f}")
    sd = eng.state_dict()                       # collective: every rank contributes its experts and shards
    if rank == 0:
        print("experts of layer 0:", tuple(sd["layers.0.moe.w13"].shape), " expert parameters on this rank:",
              eng.expert_parameters())
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
