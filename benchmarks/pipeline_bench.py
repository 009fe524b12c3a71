"""1F1B pipeline parallelism over NCCL point-to-point: how much of the activation / gradient traffic is hidden.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 --master-port 29563 \
        benchmarks/pipeline_bench.py --layers 8 --micro-batches 8 --seq 4096 --steps 5 --warmup 3

A stack of LLaMA-7B-shaped decoder layers (hidden 4096, 32 heads, SwiGLU 11008) is cut into one stage per GPU; every
micro-batch is one sequence of ``--seq`` tokens, so 32 MiB of bf16 activations cross each stage boundary per
micro-batch and direction. Two timings per rank, CUDA events, MAX over ranks:

* ``pipeline_ms``: one 1F1B pass (forward + backward of all micro-batches, gradients accumulated, no optimizer);
* ``stage_ms``: the same stage doing the same forwards and backwards on locally made inputs, no communication.

A 1F1B schedule of ``m`` micro-batches on ``s`` equal stages takes ``(m + s - 1) / m`` stage times even with free
communication (the bubble); what ``pipeline_ms`` has on top of that is exposed send/recv and scheduling overhead.
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

from ghost_flow_b200 import models as M  # noqa: E402
from ghost_flow_b200.models.llama import LLaMADecoderLayer  # noqa: E402
from ghost_flow_b200.ops import fused as ops  # noqa: E402
from ghost_flow_b200.parallel.distributed import PipelineParallel  # noqa: E402


class Stage(torch.nn.Module):
    def __init__(self, cfg, n_layers, dev):
        super().__init__()
        self.cfg = cfg
        self.layers = torch.nn.ModuleList([LLaMADecoderLayer(cfg, dev, torch.bfloat16) for _ in range(n_layers)])
        self._rope = None

    def forward(self, x):
        if self._rope is None:
            self._rope = ops.rope_tables(x.shape[1], self.cfg.head_dim, self.cfg.rope_theta, x.device)
        for layer in self.layers:
            x = layer(x, *self._rope)
        return x


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=8)
    ap.add_argument("--micro-batches", type=int, default=8)
    ap.add_argument("--seq", type=int, default=4096)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    a = ap.parse_args()
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    world = int(os.environ.get("WORLD_SIZE", 1))
    dist.init_process_group("nccl", device_id=dev)
    rank = dist.get_rank()
    cfg = M.LLaMAConfig.llama_7b()
    d, m = cfg.hidden_size, a.micro_batches
    torch.manual_seed(rank)
    stage = Stage(cfg, a.layers // world, dev)
    pp = PipelineParallel(stage, num_micro_batches=m, dtype=torch.bfloat16, device=dev,
                          activation_shape=lambda rows: (rows, a.seq, d))
    xs = [torch.randn(1, a.seq, d, device=dev, dtype=torch.bfloat16) * 0.1 for _ in range(m)]
    ys = [torch.randn(1, a.seq, d, device=dev, dtype=torch.bfloat16) * 0.1 for _ in range(m)]

    def loss_fn(out, tgt):
        return (out.float() - tgt.float()).pow(2).mean()

    def timed(fn):
        for _ in range(a.warmup):
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(a.steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / a.steps], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.item()

    def pipeline():
        stage.zero_grad(set_to_none=True)
        pp.run(xs, loss_fn, ys, rows=1)

    def alone():
        stage.zero_grad(set_to_none=True)
        for i in range(m):
            x = xs[i].detach().requires_grad_(True)
            (loss_fn(stage(x), ys[i]) / m).backward()

    stage_ms = timed(alone)
    pipe_ms = timed(pipeline)
    ideal = stage_ms * (m + world - 1) / m
    if rank == 0:
        act_mib = a.seq * d * 2 / 2 ** 20
        print(json.dumps({"metric": "pipeline_1f1b_ms", "n_gpus": world, "pipeline_ms": round(pipe_ms, 2),
                          "stage_ms": round(stage_ms, 2), "ideal_with_bubble_ms": round(ideal, 2),
                          "exposed_p2p_and_overhead_ms": round(pipe_ms - ideal, 2),
                          "fraction_of_ideal": round(ideal / pipe_ms, 3),
                          "tokens_per_s": round(m * a.seq / (pipe_ms * 1e-3), 1),
                          "config": {"layers": a.layers, "stages": world, "micro_batches": m, "seq_len": a.seq,
                                     "activation_mib_per_boundary_and_direction": act_mib, "dtype": "bf16",
                                     "p2p_batches_per_step": pp.p2p_batches}}))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
