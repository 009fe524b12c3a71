"""Mixtral training with expert parallelism = world size, one rank per GPU.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29561 \
        benchmarks/mixtral_ep_bench.py --layers 32 --micro-batch 1 --seq 4096 --steps 5 --warmup 3

Model: Mixtral-8x7B layer shapes (hidden 4096, 32 heads / 8 KV heads, 8 SwiGLU experts of 14336, top-2) with
``--layers`` decoder layers (32 = the full 46.7 B-parameter model, which needs 8 GPUs: the experts' bf16 weights, fp32
master copies and Adam moments stay on their owner, about 90 GB per GPU). Attention and norm parameters are ZeRO-3
units moved by this library's peer-memory kernels; tokens travel to their experts and back through the dispatch /
combine kernels; expert GEMMs are grouped tcgen05 kernels. Synthetic uniform token ids, random-init weights. Timed
with CUDA events between barriers, MAX over ranks. FLOPs per token counted as 6 x active parameters (attention
projections, two experts, head) plus the causal attention term.
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

from ghost_flow_b200.models.configs import MixtralConfig  # noqa: E402
from ghost_flow_b200.ops import _lib  # noqa: E402
from ghost_flow_b200.parallel.mixtral import MixtralEngine  # noqa: E402
from ghost_flow_b200.parallel.symm import FusedComm  # noqa: E402
from ghost_flow_b200.parallel.zero3 import Comm, OptimConfig  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--micro-batch", type=int, default=1)
    ap.add_argument("--seq", type=int, default=4096)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--capacity-factor", type=float, default=2.0)
    ap.add_argument("--tiny", action="store_true", help="a small configuration for a quick functional run")
    a = ap.parse_args()
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    world = int(os.environ.get("WORLD_SIZE", 1))
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    rank = dist.get_rank() if world > 1 else 0
    cfg = MixtralConfig.mixtral_8x7b()
    if a.tiny:
        cfg = MixtralConfig(vocab_size=2048, hidden_size=512, intermediate_size=1024, num_attention_heads=4,
                            num_key_value_heads=2, max_position_embeddings=max(512, a.seq))
    cfg.num_hidden_layers = a.layers
    comm = FusedComm(dev) if world > 1 else Comm()
    T = a.micro_batch * a.seq
    eng = MixtralEngine(cfg, dev, tokens_per_rank=T, optim=OptimConfig(lr=1e-4, weight_decay=0.1), comm=comm, seed=0,
                        capacity_factor=a.capacity_factor, expert_init="device")
    g = torch.Generator().manual_seed(1 + rank)

    def batch():
        ids = torch.randint(0, cfg.vocab_size, (a.micro_batch, a.seq + 1), generator=g).to(dev)
        return ids[:, :-1], ids[:, 1:]

    for _ in range(a.warmup):
        loss = eng.step(*batch())
    torch.cuda.synchronize()
    _lib.check_status(dev)
    if world > 1:
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(a.steps):
        loss = eng.step(*batch())
    e1.record()
    torch.cuda.synchronize()
    _lib.check_status(dev)
    ms = torch.tensor([e0.elapsed_time(e1) / a.steps], device=dev)
    peak = torch.tensor([torch.cuda.max_memory_allocated(dev) / 2 ** 30], device=dev)
    counts = eng.moe.expert_counts().float()
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        dist.all_reduce(peak, op=dist.ReduceOp.MAX)
        dist.all_reduce(counts)
    d, f, hd = cfg.hidden_size, cfg.intermediate_size, cfg.head_dim
    active = a.layers * (d * (cfg.num_attention_heads + 2 * cfg.num_key_value_heads) * hd + cfg.num_attention_heads * hd * d
                         + cfg.num_experts_per_tok * 3 * d * f + cfg.num_local_experts * d) + cfg.vocab_size * d
    flops_tok = 6 * active + a.layers * 6 * a.seq * cfg.num_attention_heads * hd     # causal: half of 12 * S * H * D
    tok_s = world * T / (ms.item() * 1e-3)
    if rank == 0:
        dense = sum(u.numel for u in eng.units)
        total = dense + a.layers * (cfg.num_local_experts * 3 * d * f + cfg.num_local_experts * d)
        print(json.dumps({"metric": "mixtral_ep_train_tokens_per_s", "value": round(tok_s, 1), "n_gpus": world,
                          "ms_per_step": round(ms.item(), 2), "loss": round(float(loss), 4),
                          "tflops_per_gpu": round(tok_s * flops_tok / world / 1e12, 1),
                          "peak_mem_gib": round(peak.item(), 1),
                          "expert_load_max_over_mean": round((counts.max() / counts.mean()).item(), 3),
                          "config": {"model": "mixtral-8x7b-shape" if not a.tiny else "mixtral-tiny",
                                     "layers": a.layers, "params_b": round(total / 1e9, 2),
                                     "active_params_b": round(active / 1e9, 2), "micro_batch": a.micro_batch,
                                     "seq_len": a.seq, "parallelism": f"ep{world}+zero3", "capacity_factor": a.capacity_factor,
                                     "dtype": "bf16", "data": "synthetic"}}))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
