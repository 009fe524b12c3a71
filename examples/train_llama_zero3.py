"""ZeRO-3 training of a LLaMA-shaped model with the hand-scheduled engine. One process per GPU:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 examples/train_llama_zero3.py --model llama-7b

Runs on one process and on CPU (tiny model) as well."""
import argparse
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from ghost_flow_b200.models.configs import LLaMAConfig  # noqa: E402
from ghost_flow_b200.parallel.comm import make_comm  # noqa: E402
from ghost_flow_b200.parallel.zero3 import OptimConfig, Zero3LlamaEngine  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="llama-tiny", choices=["llama-tiny", "llama-7b"])
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--seq", type=int, default=0)
    a = ap.parse_args()
    cuda = torch.cuda.is_available()
    world = int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    dev = torch.device("cuda", local) if cuda else torch.device("cpu")
    if cuda:
        torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl" if cuda else "gloo", **({"device_id": dev} if cuda else {}))
    cfg = LLaMAConfig.llama_7b() if a.model == "llama-7b" else LLaMAConfig.llama_tiny()
    seq = a.seq or (4096 if a.model == "llama-7b" else 128)
    comm = make_comm("fused" if (cuda and world > 1) else "nccl", dev)
    eng = Zero3LlamaEngine(cfg, dev, comm=comm, optim=OptimConfig(lr=3e-4, weight_decay=0.1), seed=0)
    g = torch.Generator().manual_seed(dist.get_rank() if world > 1 else 0)
    for step in range(a.steps):
        ids = torch.randint(0, cfg.vocab_size, (1, seq + 1), generator=g).to(dev)
        loss = eng.step(ids[:, :-1], ids[:, 1:])
        if (dist.get_rank() if world > 1 else 0) == 0:
            print(f"step {step} loss {float(loss):.4f}")
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
