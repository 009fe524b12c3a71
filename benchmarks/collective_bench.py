"""Fused compute + collective kernels against their NCCL-only counterparts, one rank per GPU.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port 29555 \
        benchmarks/collective_bench.py --mode tp  --tokens 16384 --hidden 8192 --ffn 28672
    ... benchmarks/collective_bench.py --mode moe --tokens 4096 --hidden 4096 --ffn 14336 --experts 8 --topk 2

Every number is timed with CUDA events on the launching stream after warm-up, between a barrier and a
synchronize on both sides, and reduced with MAX over ranks. Operands are far larger than L2 (126 MB) at the default
sizes. Rank 0 prints one JSON line per measurement. Roofline = slower of FLOPs at the measured cuBLAS bf16 rate and
bytes that must cross NVLink at 770 GB/s per direction per GPU (``MEASURED_PEAKS.json`` when present).
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

from ghost_flow_b200.ops import _lib, raw  # noqa: E402

NVLINK_GBS = 770.0


def peak_tflops():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        return json.load(open(p))["bf16_tflops"], "measured"
    return 1590.0, "fallback"


def timed(fn, iters, warmup=3):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / iters], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t)


def emit(rank, **kw):
    if rank == 0:
        print(json.dumps(kw), flush=True)


def bench_tp(a, dev, rank, world):
    from ghost_flow_b200.parallel.tp import AllGatherGemm, GemmReduceScatter

    T, H, F = a.tokens, a.hidden, a.ffn
    tf, src = peak_tflops()
    n_col = F // world                       # column-parallel: every rank owns F / world output features
    for copy_ctas in a.copy_ctas:
        ag = AllGatherGemm(T, H, dev, copy_ctas=copy_ctas)
        x = torch.randn(T // world, H, device=dev, dtype=torch.bfloat16)
        w = torch.randn(n_col, H, device=dev, dtype=torch.bfloat16) * 0.02
        fused = timed(lambda: ag(x, w), a.iters)
        nccl = timed(lambda: ag.reference(x, w), a.iters)
        flops = 2.0 * T * n_col * H
        link_bytes = 2.0 * T * H * (world - 1) / world
        roof = max(flops / tf / 1e9, link_bytes / NVLINK_GBS / 1e6)
        emit(rank, op="allgather+gemm", world=world, M=T, N=n_col, K=H, copy_ctas=copy_ctas, fused_ms=round(fused, 4),
             nccl_then_gemm_ms=round(nccl, 4), roofline_ms=round(roof, 4), frac_of_roofline=round(roof / fused, 3),
             peaks=src)
        del ag
    rs = GemmReduceScatter(T, H, dev)
    xl = torch.randn(T, n_col, device=dev, dtype=torch.bfloat16)
    wl = torch.randn(H, n_col, device=dev, dtype=torch.bfloat16) * 0.02
    fused = timed(lambda: rs(xl, wl), a.iters)
    nccl = timed(lambda: rs.reference(xl, wl), a.iters)
    flops = 2.0 * T * H * n_col
    link_bytes = 2.0 * T * H * (world - 1) / world
    roof = max(flops / tf / 1e9, link_bytes / NVLINK_GBS / 1e6)
    emit(rank, op="gemm+reduce_scatter", world=world, M=T, N=H, K=n_col, fused_ms=round(fused, 4),
         gemm_then_nccl_ms=round(nccl, 4), roofline_ms=round(roof, 4), frac_of_roofline=round(roof / fused, 3), peaks=src)
    # decode-sized problem: latency of the collective dominates
    Ts = 64 * world
    rs2 = GemmReduceScatter(Ts, H, dev)
    xs = torch.randn(Ts, n_col, device=dev, dtype=torch.bfloat16)
    emit(rank, op="gemm+reduce_scatter(small)", world=world, M=Ts, N=H, K=n_col,
         fused_ms=round(timed(lambda: rs2(xs, wl), 50), 4), gemm_then_nccl_ms=round(timed(lambda: rs2.reference(xs, wl), 50), 4))


def bench_moe(a, dev, rank, world):
    from ghost_flow_b200.parallel.ep import ExpertParallelMoE

    T, d, f, E, k = a.tokens, a.hidden, a.ffn, a.experts, a.topk
    tf, src = peak_tflops()
    moe = ExpertParallelMoE(d, f, E, k, T, dev, capacity_factor=a.capacity_factor, seed=1)
    g = torch.Generator(device="cpu").manual_seed(2)
    moe.gate_pad[:E] = (torch.randn(E, d, generator=g) * 0.05).to(torch.bfloat16).to(dev)
    torch.manual_seed(10 + rank)
    x = torch.randn(T, d, device=dev, dtype=torch.bfloat16)
    dy = torch.randn(T, d, device=dev, dtype=torch.bfloat16) * 0.1

    def fwd():
        return moe.forward(x)

    def fwd_bwd():
        y, ctx = moe.forward(x)
        moe.backward(ctx, dy)

    t_f = timed(fwd, a.iters)
    t_fb = timed(fwd_bwd, a.iters)
    torch.cuda.synchronize()
    _lib.check_status(dev)
    # NCCL-only arm: all-gather the tokens, every rank runs its experts on all tokens, reduce-scatter the outputs
    w13, w2 = moe.w13, moe.w2
    el = moe.el

    def nccl_fwd():
        xa = torch.empty(T * world, d, device=dev, dtype=torch.bfloat16)
        dist.all_gather_into_tensor(xa, x)
        logits = raw.gemm(xa, False, moe.gate_pad, True, out_dtype=torch.float32)[:, :E]
        probs = torch.softmax(logits, -1)
        top, idx = probs.topk(k, -1)
        wts = (top / top.sum(-1, keepdim=True)).to(torch.bfloat16)
        ya = torch.zeros(T * world, d, device=dev, dtype=torch.bfloat16)
        for j in range(el):
            tok, slot = (idx == rank * el + j).nonzero(as_tuple=True)
            if tok.numel() == 0:
                continue
            h = raw.gemm(xa[tok], False, w13[j], True)
            o = raw.gemm(raw.swiglu_fwd(h), False, w2[j], True)
            ya.index_add_(0, tok, o * wts[tok, slot, None])
        y = torch.empty(T, d, device=dev, dtype=torch.bfloat16)
        dist.reduce_scatter_tensor(y, ya)
        return y

    t_n = timed(nccl_fwd, max(2, a.iters // 2)) if world > 1 else None
    flops_f = 2.0 * T * k * d * 3 * f           # per rank: its tokens x k experts x (2f + f) x d x 2
    link = 2.0 * T * k * d * 2 * (world - 1) / world   # dispatch + combine rows leaving this GPU
    roof_f = max(flops_f / tf / 1e9, link / NVLINK_GBS / 1e6)
    emit(rank, op="moe_layer", world=world, tokens_per_rank=T, hidden=d, ffn=f, experts=E, topk=k, fwd_ms=round(t_f, 4),
         fwd_bwd_ms=round(t_fb, 4), nccl_allgather_fwd_ms=round(t_n, 4) if t_n else None,
         fwd_tokens_per_s=round(T * world / t_f * 1e3), fwd_bwd_tokens_per_s=round(T * world / t_fb * 1e3),
         roofline_fwd_ms=round(roof_f, 4), frac_of_roofline_fwd=round(roof_f / t_f, 3),
         frac_of_roofline_fwd_bwd=round(3 * roof_f / t_fb, 3), peaks=src)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--mode", choices=["tp", "moe"], required=True)
    ap.add_argument("--tokens", type=int, default=16384)
    ap.add_argument("--hidden", type=int, default=8192)
    ap.add_argument("--ffn", type=int, default=28672)
    ap.add_argument("--experts", type=int, default=8)
    ap.add_argument("--topk", type=int, default=2)
    ap.add_argument("--capacity-factor", type=float, default=2.0)
    ap.add_argument("--copy-ctas", type=int, nargs="+", default=[16])
    ap.add_argument("--iters", type=int, default=10)
    a = ap.parse_args()
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    rank, world = dist.get_rank(), dist.get_world_size()
    (bench_tp if a.mode == "tp" else bench_moe)(a, dev, rank, world)
    torch.cuda.synchronize()
    _lib.check_status(dev)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
