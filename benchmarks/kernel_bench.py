"""Times ONE kernel of the library on one GPU and prints a JSON line with its roofline fraction.

    python benchmarks/kernel_bench.py --kernel gemm_nt --m 8192 --n 8192 --k 8192
    python benchmarks/kernel_bench.py --kernel attn_fwd --batch 2 --seq 4096 --heads 32 --dim 128
    python benchmarks/kernel_bench.py --kernel rmsnorm_fwd --rows 32768 --cols 4096

Timing: CUDA events on the launching stream, ``--warmup`` untimed launches, a write of a buffer larger than L2
between timed launches (so every launch starts with a cold L2), median over ``--iters``. The roofline
denominators come from ``MEASURED_PEAKS.json`` at the repository root when it exists (a copy bandwidth and a
cuBLAS bf16 rate measured on the same pool); otherwise 6650 GB/s and 1590 TFLOP/s are used and reported as
"fallback". ``--iters 1 --warmup 1 --no-flush`` is the shape used for a profiler capture.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from ghost_flow_b200.ops import _lib, raw  # noqa: E402
from ghost_flow_b200.ops.gemm import gemm_raw  # noqa: E402


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return d["hbm_gbs"], d["bf16_tflops"], "measured"
    return 6650.0, 1590.0, "fallback"


def build(args, dev):
    """Returns (fn, flops, bytes) for the chosen kernel."""
    bf = torch.bfloat16
    k = args.kernel
    if k in ("gemm_nt", "gemm_nn", "gemm_tn"):
        M, N, K = args.m, args.n, args.k
        a = torch.randn((K, M) if k == "gemm_tn" else (M, K), device=dev, dtype=bf)
        b = torch.randn((K, N) if k in ("gemm_nn", "gemm_tn") else (N, K), device=dev, dtype=bf)
        out = torch.empty(M, N, device=dev, dtype=bf)
        fn = lambda: gemm_raw(a, k == "gemm_tn", b, k in ("gemm_nn", "gemm_tn"), M, N, K, out=out)  # noqa: E731
        return fn, 2.0 * M * N * K, 2.0 * (M * K + N * K + M * N)
    if k == "gemm_skinny":
        M, N, K = args.m, args.n, args.k
        a = torch.randn(M, K, device=dev, dtype=bf)
        b = torch.randn(N, K, device=dev, dtype=bf)
        return (lambda: gemm_raw(a, False, b, False, M, N, K)), 2.0 * M * N * K, 2.0 * (M * K + N * K + M * N)
    if k == "cublas_nt":
        M, N, K = args.m, args.n, args.k
        a = torch.randn(M, K, device=dev, dtype=bf)
        b = torch.randn(N, K, device=dev, dtype=bf)
        out = torch.empty(M, N, device=dev, dtype=bf)
        return (lambda: torch.matmul(a, b.t(), out=out)), 2.0 * M * N * K, 2.0 * (M * K + N * K + M * N)
    if k in ("gemm_fp8_rowcol", "gemm_fp8_block"):
        from ghost_flow_b200.ops import fp8
        M, N, K = args.m, args.n, args.k
        mode = 0 if k == "gemm_fp8_rowcol" else 1
        a = torch.randn(M, K, device=dev, dtype=bf)
        b = torch.randn(N, K, device=dev, dtype=bf)
        aq, sa = fp8.quantize_rows(a, mode)
        bq, sb = fp8.quantize_rows(b, 0) if mode == 0 else fp8.quantize_block128(b)
        out = torch.empty(M, N, device=dev, dtype=bf)
        return (lambda: fp8.gemm_fp8(aq, sa, bq, sb, mode, out=out)), 2.0 * M * N * K, 1.0 * (M * K + N * K) + 2.0 * M * N
    if k == "gemm_fp8_skinny":
        from ghost_flow_b200.ops import fp8
        M, N, K = args.m, args.n, args.k
        aq, sa = fp8.quantize_rows(torch.randn(M, K, device=dev, dtype=bf), 0)
        bq, sb = fp8.quantize_rows(torch.randn(N, K, device=dev, dtype=bf), 0)
        out = torch.empty(M, N, device=dev, dtype=bf)
        return (lambda: fp8.gemm_fp8(aq, sa, bq, sb, 0, out=out)), 2.0 * M * N * K, 1.0 * (M * K + N * K) + 2.0 * M * N
    if k == "quant_fp8_rows":
        from ghost_flow_b200.ops import fp8
        x = torch.randn(args.rows, args.cols, device=dev, dtype=bf)
        return (lambda: fp8.quantize_rows(x, 1)), 0.0, 3.0 * args.rows * args.cols
    if k == "attn_decode":
        B, S, H, Hkv, D = args.batch, args.seq, args.heads, args.kv_heads or args.heads, args.dim
        q = torch.randn(B, H * D, device=dev, dtype=bf)
        kc = torch.randn(B, S, Hkv * D, device=dev, dtype=bf)
        vc = torch.randn(B, S, Hkv * D, device=dev, dtype=bf)
        return (lambda: raw.attn_decode(q, kc, vc, S, B, H, Hkv, D)), 4.0 * B * H * S * D, 4.0 * B * S * Hkv * D
    if k in ("attn_fwd", "attn_bwd"):
        B, S, H, Hkv, D = args.batch, args.seq, args.heads, args.kv_heads or args.heads, args.dim
        q = torch.randn(B * S, H * D, device=dev, dtype=bf)
        kk = torch.randn(B * S, Hkv * D, device=dev, dtype=bf)
        v = torch.randn(B * S, Hkv * D, device=dev, dtype=bf)
        flops_f = 4.0 * B * H * S * S * D * 0.5
        if k == "attn_fwd":
            return (lambda: raw.attn_fwd(q, kk, v, B, S, H, Hkv, D, True)), flops_f, 2.0 * (2 * q.numel() + 2 * kk.numel())
        o, lse = raw.attn_fwd(q, kk, v, B, S, H, Hkv, D, True)
        do = torch.randn_like(o)
        dq, dk, dv = torch.empty_like(q), torch.empty_like(kk), torch.empty_like(v)
        fn = lambda: raw.attn_bwd(q, kk, v, o, do, lse, dq, dk, dv, B, S, H, Hkv, D, True)  # noqa: E731
        return fn, 2.5 * flops_f, 2.0 * (4 * q.numel() + 4 * kk.numel()) + 8.0 * q.numel()
    R, C = args.rows, args.cols
    if k == "rmsnorm_fwd":
        x = torch.randn(R, C, device=dev, dtype=bf)
        w = torch.ones(C, device=dev, dtype=bf)
        return (lambda: raw.rmsnorm_fwd(x, w, 1e-5)), 0.0, 4.0 * R * C
    if k == "rmsnorm_bwd":
        x = torch.randn(R, C, device=dev, dtype=bf)
        w = torch.ones(C, device=dev, dtype=bf)
        dy = torch.randn_like(x)
        _, rstd, _ = raw.rmsnorm_fwd(x, w, 1e-5)
        return (lambda: raw.rmsnorm_bwd(x, w, dy, rstd)), 0.0, 6.0 * R * C
    if k == "rope":
        H, D = args.heads, args.dim
        x = torch.randn(R, H, D, device=dev, dtype=bf)
        from ghost_flow_b200.ops.fused import rope_tables
        cos, sin = rope_tables(args.seq, D, 10000.0, dev)
        return (lambda: raw.rope_(x, cos, sin, args.seq)), 0.0, 4.0 * R * H * D
    if k == "swiglu_bwd":
        gu = torch.randn(R, 2 * C, device=dev, dtype=bf)
        dy = torch.randn(R, C, device=dev, dtype=bf)
        return (lambda: raw.swiglu_bwd(gu, dy)), 0.0, 10.0 * R * C
    if k in ("add_f32", "relu_f32", "softmax_f32", "sum_f32"):
        from ghost_flow_b200.ops import elementwise as ew
        if k == "softmax_f32":
            x = torch.randn(R, C, device=dev)
            return (lambda: ew.softmax_rows(x)), 0.0, 8.0 * R * C
        x, y = torch.randn(R * C, device=dev), torch.randn(R * C, device=dev)
        if k == "add_f32":
            return (lambda: ew.binary(x, y, "add")), 0.0, 12.0 * R * C
        if k == "sum_f32":
            return (lambda: ew.reduce_all(x, "sum")), 0.0, 4.0 * R * C
        return (lambda: ew.unary_any(x, "relu")), 0.0, 8.0 * R * C
    if k == "split_bf16":
        from ghost_flow_b200.ops.gemm import matmul_fp32_split
        M, N, K = args.m, args.n, args.k
        a, b = torch.randn(M, K, device=dev), torch.randn(K, N, device=dev)
        return (lambda: matmul_fp32_split(a, b)), 2.0 * M * N * K, 4.0 * (M * K + N * K + M * N)
    if k in ("im2col_nhwc", "conv_nhwc", "conv_unfolded", "pad_nhwc"):
        # --batch images of --rows x --rows pixels, --cols channels in and out, 3 x 3 window, stride 1
        from ghost_flow_b200.ops.render import conv2d_nhwc, im2col_nhwc, pack_conv_weight_nhwc
        B, HW, Cc = args.batch, args.rows, args.cols
        x = torch.randn(B, HW, HW, Cc, device=dev, dtype=bf)
        w = torch.randn(Cc, Cc, 3, 3, device=dev) / (3.0 * Cc ** 0.5)
        wp, bp = pack_conv_weight_nhwc(w, torch.zeros(Cc, device=dev))
        px = B * HW * HW
        if k == "im2col_nhwc":
            return (lambda: im2col_nhwc(x, 3, 3, 1, 1)), 0.0, 2.0 * px * Cc * 10
        if k == "pad_nhwc":
            from ghost_flow_b200.ops.render import pad_nhwc
            return (lambda: pad_nhwc(x, 1)), 0.0, 2.0 * Cc * (px + B * (HW + 1) * (HW + 1))
        if k == "conv_unfolded":      # gather + GEMM even where the implicit path applies
            from ghost_flow_b200.ops import render
            render.IMPLICIT_CONV = False
        return (lambda: conv2d_nhwc(x, wp, bp, (3, 3), 1, 1, relu=True)), 2.0 * px * Cc * Cc * 9, \
            2.0 * (2 * px * Cc + 9 * Cc * Cc)
    if k == "layernorm":
        from ghost_flow_b200.ops import fused
        x = torch.randn(R, C, device=dev, dtype=bf)
        w, b = torch.ones(C, device=dev, dtype=bf), torch.zeros(C, device=dev, dtype=bf)
        return (lambda: fused.layer_norm(x, w, b, 1e-5)), 0.0, 4.0 * R * C
    if k == "moe_layer":
        from ghost_flow_b200.parallel.ep import ExpertParallelMoE
        T, d, f = args.rows, args.cols, args.k
        moe = ExpertParallelMoE(d, f, 8, 2, T, dev, seed=1)
        moe.gate_pad[:8] = (torch.randn(8, d, device=dev) * 0.05).to(bf)
        x = torch.randn(T, d, device=dev, dtype=bf)
        dy = torch.randn(T, d, device=dev, dtype=bf) * 0.1

        def step():
            y, ctx = moe.forward(x)
            moe.backward(ctx, dy)
        return step, 2.0 * T * 2 * d * 3 * f * 3, 2.0 * 8 * 3 * d * f * 3
    if k == "swiglu_fwd":
        gu = torch.randn(R, 2 * C, device=dev, dtype=bf)
        return (lambda: raw.swiglu_fwd(gu)), 0.0, 6.0 * R * C
    if k == "xent":
        logits = torch.randn(R, C, device=dev, dtype=bf)
        tgt = torch.randint(0, C, (R,), device=dev)
        return (lambda: raw.xent_fwd_bwd(logits, tgt)), 0.0, 4.0 * R * C
    if k == "adamw":
        n = R * C
        p32 = torch.randn(n, device=dev)
        m, v = torch.zeros_like(p32), torch.zeros_like(p32)
        g = torch.randn(n, device=dev, dtype=bf)
        plp = torch.empty(n, device=dev, dtype=bf)
        fn = lambda: raw.adamw_flat(p32, m, v, g, plp, lr=1e-3, beta1=0.9, beta2=0.95, eps=1e-8,  # noqa: E731
                                    weight_decay=0.1, step=3)
        return fn, 0.0, n * (3 * 4 * 2 + 2 + 2.0)
    raise SystemExit(f"unknown kernel {k}")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--kernel", required=True)
    ap.add_argument("--m", type=int, default=8192)
    ap.add_argument("--n", type=int, default=8192)
    ap.add_argument("--k", type=int, default=8192)
    ap.add_argument("--batch", type=int, default=2)
    ap.add_argument("--seq", type=int, default=4096)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=0)
    ap.add_argument("--dim", type=int, default=128)
    ap.add_argument("--rows", type=int, default=32768)
    ap.add_argument("--cols", type=int, default=4096)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--no-flush", action="store_true")
    args = ap.parse_args()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    torch.manual_seed(0)
    fn, flops, nbytes = build(args, dev)
    flush = None if args.no_flush else torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    for _ in range(args.warmup):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(args.iters):
        if flush is not None:
            flush.fill_(1)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
    _lib.check_status(dev)
    ms = statistics.median(times)
    hbm, tf, src = peaks()
    res = {"kernel": args.kernel, "ms": round(ms, 5), "min_ms": round(min(times), 5), "peaks": src,
           "l2_flush": flush is not None,
           "args": {k: v for k, v in vars(args).items() if k not in ("kernel", "iters", "warmup", "no_flush")}}
    if flops:
        res["tflops"] = round(flops / ms / 1e9, 1)
        res["frac_of_gemm_peak"] = round(flops / ms / 1e9 / tf, 3)
    res["gbs"] = round(nbytes / ms / 1e6, 1)
    res["frac_of_copy_bw"] = round(nbytes / ms / 1e6 / hbm, 3)
    print(json.dumps(res))


if __name__ == "__main__":
    main()
