"""Re-measures, on one B200, the micro-benchmarks that the reference publishes tables for.

The reference ships no program that produces its tables (ghost-flow-py/PERFORMANCE.md:137-141 points at an
``examples/benchmark.py`` that does not exist), states no hardware for them and cannot be built offline, so its
figures are carried along as ``published_ms`` for orientation only; what this program measures is this framework,
through its public API (``ghost_flow_b200.Tensor``, ``nn`` layers, ``models``), next to the vendor-library path
(``torch`` fp32 / cuDNN) on the same GPU:

* square matmul 256 / 512 / 1024 / 2048 (PERFORMANCE.md:34-40, DOCS/PERFORMANCE_SUMMARY.md:34-39),
* element-wise ops over 10 M elements (PERFORMANCE.md:57-62),
* a ResNet-50 3 x 3 convolution and the fused Conv+BN+ReLU (DOCS/PERFORMANCE_SUMMARY.md:43-46); the reference does
  not say which layer or batch: conv3_x (128 -> 128 channels, 28 x 28) at batch 32 is used,
* ResNet-18 training, scaled to one epoch (PERFORMANCE.md:46-51); dataset unstated there: 50 000 images of
  3 x 32 x 32 at batch 128, SGD with momentum, bf16 autocast,
* BERT-base inference latency per batch (PERFORMANCE.md:92-100); batch unstated there: 32 sequences of 128 tokens.

    python benchmarks/published_table_bench.py [--iters 20] [--warmup 5] [--only matmul,elementwise,conv,resnet18,bert]

Timing: CUDA events on the launching stream, median over ``--iters`` launches after ``--warmup`` untimed ones; a
buffer larger than L2 is rewritten before every timed launch so that none of these small working sets is served
from cache. One JSON line per row.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys

import torch
import torch.nn.functional as F

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import ghost_flow_b200 as gf  # noqa: E402
from ghost_flow_b200 import models, nn, optim  # noqa: E402
from ghost_flow_b200.ops import _lib  # noqa: E402

DEV = "cuda"
_FLUSH = None


def timed(fn, iters: int, warmup: int, flush: bool = True) -> float:
    """Median milliseconds of ``fn()``."""
    global _FLUSH
    if flush and _FLUSH is None:
        _FLUSH = torch.empty(256 << 20, dtype=torch.uint8, device=DEV)
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        if flush:
            _FLUSH.fill_(1)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        ts.append(a.elapsed_time(b))
    return statistics.median(ts)


def emit(**row):
    row["launches_from_libgfb200"] = _lib.launch_count() if hasattr(_lib, "launch_count") else None
    print(json.dumps(row), flush=True)


def bench_matmul(args):
    published = {256: (0.8, None), 512: (3.2, None), 1024: (12.3, 2.1), 2048: (52.1, None)}
    for n, (summary_ms, perf_md_ms) in published.items():
        a32, b32 = torch.randn(n, n, device=DEV), torch.randn(n, n, device=DEV)
        ta, tb = gf.Tensor(a32.bfloat16()), gf.Tensor(b32.bfloat16())
        ours = timed(lambda: ta.matmul(tb), args.iters, args.warmup)
        ours_warm = timed(lambda: ta.matmul(tb), args.iters, args.warmup, flush=False)
        lib32 = timed(lambda: torch.matmul(a32, b32), args.iters, args.warmup)
        t32a, t32b = gf.Tensor(a32), gf.Tensor(b32)
        split = timed(lambda: t32a.matmul(t32b), args.iters, args.warmup)
        ref = a32.double() @ b32.double()
        split_err = float((t32a.matmul(t32b).data.double() - ref).abs().max() / ref.abs().max())
        # ours_idle_gpu_ms: same call issued to an idle GPU, where the host-side launch path is what is timed
        emit(bench=f"matmul_{n}x{n}", ours_ms=ours, ours_idle_gpu_ms=ours_warm,
             ours_dtype="bf16 in, fp32 accumulate (tcgen05 kernel)", ours_tflops=2.0 * n ** 3 / ours / 1e9,
             ours_fp32_in_out_ms=split, ours_fp32_in_out_max_rel_err=split_err,
             ours_fp32_in_out_how="same kernel over hi/lo bf16 splits of fp32 operands (3x contraction)",
             library_fp32_ms=lib32,
             published_ms={"DOCS/PERFORMANCE_SUMMARY.md": summary_ms, "ghost-flow-py/PERFORMANCE.md": perf_md_ms},
             published_dtype="fp32, hardware not stated")


def bench_elementwise(args):
    n = 10_000_000
    x32, y32 = torch.randn(n, device=DEV), torch.randn(n, device=DEV)
    tx, ty = gf.Tensor(x32), gf.Tensor(y32)
    rows = {"add": (lambda: tx + ty, 12 * n), "mul": (lambda: tx * ty, 12 * n), "relu": (lambda: tx.relu(), 8 * n),
            "sigmoid": (lambda: tx.sigmoid(), 8 * n), "gelu": (lambda: tx.gelu(), 8 * n)}
    for name, (fn, nbytes) in rows.items():
        ms = timed(fn, args.iters, args.warmup)
        emit(bench=f"elementwise_{name}_10M_fp32", ours_ms=ms, ours_gbs=nbytes / ms / 1e6,
             published_ms={"ghost-flow-py/PERFORMANCE.md": 1.2}, published_dtype="fp32, op and hardware not stated")


def bench_conv(args):
    N, C, H, W, Co, k = 32, 128, 28, 28, 128, 3
    x = torch.randn(N, C, H, W, device=DEV)
    conv, bn = nn.Conv2d(C, Co, k, 1, 1).to(DEV), nn.BatchNorm2d(Co).to(DEV)
    bn.eval()
    flops = 2.0 * N * H * W * Co * C * k * k
    with torch.no_grad():
        from ghost_flow_b200.ops.render import conv2d_nhwc, pack_conv_weight_nhwc

        wp, bp = pack_conv_weight_nhwc(conv.weight, conv.bias)
        xn = x.permute(0, 2, 3, 1).contiguous().bfloat16()
        ms_conv = timed(lambda: conv2d_nhwc(xn, wp, bp, (k, k), 1, 1, relu=False), args.iters, args.warmup)
        fused = nn.ConvBNReLU(conv, bn)
        w2, b2 = pack_conv_weight_nhwc(fused.weight, fused.bias)
        ms_fused = timed(lambda: conv2d_nhwc(xn, w2, b2, (k, k), 1, 1, relu=True), args.iters, args.warmup)
        ms_fused_nchw = timed(lambda: fused(x), args.iters, args.warmup)
        lib_conv = timed(lambda: F.conv2d(x, conv.weight, conv.bias, 1, 1), args.iters, args.warmup)
        lib_chain = timed(lambda: torch.relu(bn(conv(x))), args.iters, args.warmup)
        xcl = x.bfloat16().contiguous(memory_format=torch.channels_last)
        wcl = conv.weight.bfloat16().contiguous(memory_format=torch.channels_last)
        bcl = conv.bias.bfloat16()
        lib_bf16 = timed(lambda: F.conv2d(xcl, wcl, bcl, 1, 1), args.iters, args.warmup)
    shape = f"batch {N}, {C}->{Co} channels, {H}x{W}, {k}x{k}"
    emit(bench="conv2d_resnet50_conv3x", shape=shape, ours_ms=ms_conv, ours_tflops=flops / ms_conv / 1e9,
         ours_dtype="bf16 channels-last: gather kernel + tcgen05 GEMM", library_fp32_nchw_ms=lib_conv,
         library_bf16_channels_last_ms=lib_bf16, published_ms={"DOCS/PERFORMANCE_SUMMARY.md": 8.4})
    emit(bench="conv_bn_relu_fused", shape=shape, ours_ms=ms_fused, ours_nchw_fp32_io_ms=ms_fused_nchw,
         ours_tflops=flops / ms_fused / 1e9, library_unfused_fp32_ms=lib_chain,
         published_ms={"DOCS/PERFORMANCE_SUMMARY.md": 9.2})


def bench_resnet18(args):
    torch.manual_seed(0)
    batch, images = 128, 50_000
    m = models.resnet18(10, small_input=True).to(DEV).to(memory_format=torch.channels_last)
    opt = optim.SGD(m.parameters(), lr=0.05, momentum=0.9, weight_decay=5e-4)
    host_x = torch.randn(batch, 3, 32, 32).pin_memory()
    host_y = torch.randint(0, 10, (batch,)).pin_memory()

    def step():
        x = host_x.to(DEV, non_blocking=True).contiguous(memory_format=torch.channels_last)
        y = host_y.to(DEV, non_blocking=True)
        opt.zero_grad()
        with torch.autocast("cuda", dtype=torch.bfloat16):
            loss = F.cross_entropy(m(x).float(), y)
        loss.backward()
        opt.step()
        return loss

    ms = timed(step, max(args.iters // 2, 5), args.warmup, flush=False)
    steps = (images + batch - 1) // batch
    emit(bench="resnet18_train_epoch", shape=f"{images} images 3x32x32, batch {batch}, SGD momentum, bf16 autocast",
         ours_ms_per_step=ms, ours_epoch_s=ms * steps / 1e3, ours_images_per_s=batch / ms * 1e3,
         published_s={"ghost-flow-py/PERFORMANCE.md": 45.0}, note="dataset, batch and hardware not stated by the reference")
    m.eval()
    engine = m.compile_inference()
    xi = torch.randn(256, 3, 32, 32, device=DEV)
    with torch.no_grad():
        ms_e = timed(lambda: engine(xi), args.iters, args.warmup, flush=False)
        ms_l = timed(lambda: m(xi), args.iters, args.warmup, flush=False)
        graphed = m.compile_inference(cuda_graph=True)
        ms_g = timed(lambda: graphed(xi), args.iters, args.warmup, flush=False)
    emit(bench="resnet18_inference_batch256", ours_engine_ms=ms_e, ours_engine_cuda_graph_ms=ms_g,
         ours_images_per_s=256 / min(ms_e, ms_g) * 1e3, library_fp32_eager_ms=ms_l)
    m50 = models.resnet50(1000).to(DEV).eval()
    e50 = m50.compile_inference()
    x50 = torch.randn(64, 3, 224, 224, device=DEV)
    with torch.no_grad():
        ms50 = timed(lambda: e50(x50), max(args.iters // 2, 5), args.warmup, flush=False)
        m50cl = m50.to(memory_format=torch.channels_last)
        x50cl = x50.contiguous(memory_format=torch.channels_last)

        def lib50():
            with torch.autocast("cuda", dtype=torch.bfloat16):
                return m50cl(x50cl)

        ms50l = timed(lib50, max(args.iters // 2, 5), args.warmup, flush=False)
        g50 = m50.compile_inference(cuda_graph=True)
        ms50g = timed(lambda: g50(x50), max(args.iters // 2, 5), args.warmup, flush=False)
    emit(bench="resnet50_inference_batch64_224", ours_engine_ms=ms50, ours_engine_cuda_graph_ms=ms50g, ours_images_per_s=64 / ms50 * 1e3,
         library_bf16_channels_last_autocast_ms=ms50l, peak_alloc_mb=torch.cuda.max_memory_allocated() / 2 ** 20,
         published_memory_mb={"DOCS/PERFORMANCE_SUMMARY.md": 892})


def bench_bert(args):
    torch.manual_seed(0)
    cfg = models.BertConfig.bert_base() if hasattr(models.BertConfig, "bert_base") else models.BertConfig()
    m = models.BertModel(cfg).to(DEV).to(torch.bfloat16).eval()
    ids = torch.randint(0, cfg.vocab_size, (32, 128), device=DEV)
    with torch.no_grad():
        ms_eager = timed(lambda: m(ids), args.iters, args.warmup, flush=False)
        runner = nn.CudaGraphRunner(lambda t: m(t).last_hidden_state, clone_outputs=False)
        ms = timed(lambda: runner(ids), args.iters, args.warmup, flush=False)
    emit(bench="bert_base_inference", shape="batch 32 x 128 tokens, bf16", ours_ms_per_batch=ms,
         ours_eager_ms_per_batch=ms_eager, ours_sequences_per_s=32 / ms * 1e3, params=sum(p.numel() for p in m.parameters()),
         peak_alloc_mb=torch.cuda.max_memory_allocated() / 2 ** 20,
         published_ms={"ghost-flow-py/PERFORMANCE.md": 15.0}, published_memory_gb=4.2,
         note="batch, sequence length and hardware not stated by the reference")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--only", default="matmul,elementwise,conv,resnet18,bert")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    table = {"matmul": bench_matmul, "elementwise": bench_elementwise, "conv": bench_conv,
             "resnet18": bench_resnet18, "bert": bench_bert}
    for name in args.only.split(","):
        torch.cuda.reset_peak_memory_stats()
        table[name.strip()](args)


if __name__ == "__main__":
    main()
