"""Tensor-parallel LLaMA inference: prefill and greedy-decode throughput, one rank per GPU.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29556 \
        benchmarks/tp_inference_bench.py --model llama-70b --batch 64 --prompt 2048 --new 256 --linear fused

Random-init weights of the named architecture generated shard by shard on the device, synthetic uniform token ids.
Timed with CUDA events between barriers, MAX over ranks: the prefill of the whole batch (includes writing the KV cache
and the first sampled token) and ``--new - 1`` decode steps. ``--layers`` overrides the depth (a shallower model of
the same width is a different, smaller config and is labelled as such in the output).
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

from ghost_flow_b200.models.configs import LLaMAConfig  # noqa: E402
from ghost_flow_b200.ops import _lib  # noqa: E402
from ghost_flow_b200.parallel.tp_inference import TPLlamaInference  # noqa: E402

MODELS = {
    "llama-70b": dict(vocab_size=32000, hidden_size=8192, intermediate_size=28672, num_hidden_layers=80,
                      num_attention_heads=64, num_key_value_heads=8, max_position_embeddings=4096),
    "llama-7b": dict(),
    "llama-tiny": dict(vocab_size=1024, hidden_size=512, intermediate_size=1024, num_hidden_layers=2,
                       num_attention_heads=8, num_key_value_heads=8, max_position_embeddings=4096),
}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="llama-70b", choices=list(MODELS))
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--prompt", type=int, default=2048)
    ap.add_argument("--new", type=int, default=256)
    ap.add_argument("--linear", default="fused", choices=["fused", "nccl", "fp8"])
    ap.add_argument("--graph", type=int, default=1, help="replay the decode step from a CUDA graph")
    ap.add_argument("--decode", default="oneshot", choices=["oneshot", "sp"],
                    help="oneshot: replicated activations, all-reduce+residual+RMSNorm in one kernel; sp: sequence-parallel")
    a = ap.parse_args()
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if int(os.environ.get("WORLD_SIZE", 1)) > 1:
        dist.init_process_group("nccl", device_id=dev)
    world = dist.get_world_size() if dist.is_initialized() else 1
    rank = dist.get_rank() if dist.is_initialized() else 0
    kw = dict(MODELS[a.model])
    if a.layers:
        kw["num_hidden_layers"] = a.layers
    cfg = LLaMAConfig(**kw)
    eng = TPLlamaInference(cfg, a.batch, a.prompt, a.new, dev, linear=a.linear, seed=0, decode=a.decode)
    ids = torch.randint(0, cfg.vocab_size, (a.batch, a.prompt), generator=torch.Generator().manual_seed(0)).to(dev)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()

    def maxms(ms):
        t = torch.tensor([ms], device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t)

    tok = eng.prefill(ids)              # warm-up (also allocates everything)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    tok = eng.prefill(ids)
    e1.record()
    barrier()
    prefill_ms = maxms(e0.elapsed_time(e1))
    steps = a.new - 1 - 3
    if a.graph:
        eng.capture_decode()
        eng.graph_decode(tok, a.prompt, 3)          # warm-up replays
        barrier()
        e0.record()
        for _ in range(steps):
            eng.graph.replay()
        e1.record()
    else:
        for t in range(3):                  # decode warm-up
            tok = eng.decode_step(tok, a.prompt + t)
        barrier()
        e0.record()
        for t in range(3, a.new - 1):
            tok = eng.decode_step(tok, a.prompt + t)
        e1.record()
    barrier()
    decode_ms = maxms(e0.elapsed_time(e1)) / steps
    _lib.check_status(dev)
    if rank == 0:
        params = sum(p.numel() if torch.is_tensor(p) else p[0].numel() for L in eng.layers for p in L.values()) * world
        print(json.dumps({"model": a.model, "layers": cfg.num_hidden_layers, "tp": world, "linear": a.linear, "batch": a.batch,
                          "prompt_len": a.prompt, "decode_steps_timed": steps, "cuda_graph": bool(a.graph), "decode": "oneshot" if eng.oneshot else "sp", "block_params": params,
                          "prefill_ms": round(prefill_ms, 2), "prefill_tokens_per_s": round(a.batch * a.prompt / prefill_ms * 1e3),
                          "decode_ms_per_step": round(decode_ms, 3), "decode_tokens_per_s": round(a.batch / decode_ms * 1e3),
                          "data": "synthetic token ids, random-init weights", "dtype": "fp8 e4m3 weights+activations" if a.linear == "fp8" else "bf16"}))
    if world > 1:
        dist.barrier()
    sys.stdout.flush()
    os._exit(0)      # a process group that took part in a graph capture can stall in its destructor


if __name__ == "__main__":
    main()
