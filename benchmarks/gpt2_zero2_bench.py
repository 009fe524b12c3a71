"""GPT-2 training with ZeRO-2 (gradients and optimizer state sharded, parameters replicated), one rank per GPU.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29557 \
        benchmarks/gpt2_zero2_bench.py --model gpt2-small --global-batch 64 --seq 1024 --steps 10 --warmup 3

The model is the model zoo's GPT (autograd over this library's kernels: tcgen05 GEMMs, FlashAttention, LayerNorm,
GELU, fused cross-entropy); the optimizer is :class:`ghost_flow_b200.parallel.distributed.ZeRoOptimizer` at stage 2:
per bucket one reduce-scatter of the flat bf16 gradient, the flat AdamW kernel on the owned shard (fp32 master +
moments, bf16 copy written in the same pass), one all-gather of the updated parameters. Synthetic uniform token ids,
random-init weights, targets = inputs shifted by one. Timed with CUDA events between barriers, MAX over ranks.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from ghost_flow_b200.models.configs import GPTConfig  # noqa: E402
from ghost_flow_b200.models.gpt import GPTForCausalLM  # noqa: E402
from ghost_flow_b200.ops import _lib  # noqa: E402
from ghost_flow_b200.parallel.distributed import ZeRoConfig, ZeRoOptimizer, ZeRoStage  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="gpt2-small", choices=["gpt2-small", "gpt2-medium", "gpt2-tiny"])
    ap.add_argument("--global-batch", type=int, default=64)
    ap.add_argument("--seq", type=int, default=1024)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--stage", type=int, default=2)
    ap.add_argument("--comm", default="nccl", choices=["nccl", "fused"],
                    help="fused: gradient reduce-scatter + AdamW in one peer-memory kernel, pull all-gather")
    ap.add_argument("--graph", action="store_true",
                    help="record zero_grad + forward + backward + optimizer step once in a CUDA graph and replay it")
    ap.add_argument("--no-overlap", action="store_true", help="run the collectives after backward, not from hooks")
    a = ap.parse_args()
    cuda = torch.cuda.is_available()
    local = int(os.environ.get("LOCAL_RANK", 0))
    dev = torch.device("cuda", local) if cuda else torch.device("cpu")
    if cuda:
        torch.cuda.set_device(local)
    world = int(os.environ.get("WORLD_SIZE", 1))
    if world > 1:
        dist.init_process_group("nccl" if cuda else "gloo", **({"device_id": dev} if cuda else {}))
    rank = dist.get_rank() if world > 1 else 0
    cfg = {"gpt2-small": GPTConfig.gpt2_small(), "gpt2-medium": GPTConfig.gpt2_medium(),
           "gpt2-tiny": GPTConfig(vocab_size=512, n_positions=128, n_embd=64, n_layer=2, n_head=4, n_inner=256)}[a.model]
    cfg.dropout = 0.0
    torch.manual_seed(0)
    model = GPTForCausalLM(cfg)
    model = model.to(dev, torch.bfloat16 if cuda else torch.float32)
    opt = ZeRoOptimizer(model.parameters(), ZeRoConfig(stage=ZeRoStage(a.stage), world_size=world, rank=rank, lr=3e-4,
                                                       betas=(0.9, 0.95), weight_decay=0.1, bucket_size=50_000_000),
                        comm=a.comm if (cuda and world > 1) else "nccl", overlap=False if a.no_overlap else None,
                        capturable=a.graph)
    mb = a.global_batch // world
    g = torch.Generator().manual_seed(1 + rank)

    def batch():
        ids = torch.randint(0, cfg.vocab_size, (mb, a.seq + 1), generator=g)
        return ids[:, :-1].to(dev), ids[:, 1:].to(dev)

    def train(x, y):
        opt.zero_grad()
        out = model(x, labels=y)
        loss = out[0] if isinstance(out, tuple) else out
        loss.backward()
        opt.step()
        return loss.detach()

    if a.graph:
        from ghost_flow_b200.utils import GraphedStep

        train = GraphedStep(train, batch(), warmup=3)

    def step():
        return train(*batch())

    for _ in range(a.warmup):
        loss = step()
    if cuda:
        torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    if cuda:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
    import time
    t0 = time.perf_counter()
    for _ in range(a.steps):
        loss = step()
    if cuda:
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / a.steps
    else:
        ms = (time.perf_counter() - t0) * 1e3 / a.steps
    t = torch.tensor([ms], device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    if cuda:
        _lib.check_status(dev)
    if rank == 0:
        n_params = sum(p.numel() for p in model.parameters())
        print(json.dumps({"metric": "GPT-2 ZeRO-%d train tokens/s" % a.stage, "model": a.model, "params": n_params, "n_gpus": world,
                          "global_batch": a.global_batch, "seq_len": a.seq, "comm": a.comm if world > 1 else "none", "cuda_graph": bool(a.graph and cuda),
                          "overlap": bool(opt.overlap), "ms_per_step": round(float(t), 3),
                          "value": round(a.global_batch * a.seq / float(t) * 1e3), "unit": "tokens/s",
                          "loss": round(float(loss), 4), "dtype": "bf16" if cuda else "fp32",
                          "memory_savings_ratio": round(opt.memory_savings_ratio(), 2),
                          "data": "synthetic uniform token ids, random-init weights"}))
    if a.graph:
        train.release()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
