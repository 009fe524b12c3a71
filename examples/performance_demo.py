"""Fusion analysis, pooled staging memory, profiling and benchmarking helpers
(the reference's examples/performance_demo.rs), on the GPU when there is one."""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from ghost_flow_b200 import utils as U  # noqa: E402


def main():
    eng = U.FusionEngine()
    ops = ["Conv2d", "BatchNorm2d", "ReLU", "Linear", "ReLU", "Softmax", "CrossEntropy"]
    for item in eng.fuse(ops):
        print("fusable at", item["index"], item["pattern"], "->", item["kernel"])
    pool = U.MemoryPool()
    bufs = [pool.allocate(1 << 16) for _ in range(4)]
    for b in bufs:
        pool.deallocate(b)
    for _ in range(4):
        pool.deallocate(pool.allocate(60000))
    print("pool reuse rate", round(pool.get_stats().reuse_rate(), 2))
    dev = "cuda" if torch.cuda.is_available() else "cpu"
    a = torch.randn(1024, 1024, device=dev, dtype=torch.bfloat16 if dev == "cuda" else torch.float32)
    prof = U.Profiler(use_cuda_events=dev == "cuda")
    for _ in range(3):
        with prof.start("matmul_1024"):
            (a @ a)
    print({k: round(v["avg_ms"], 4) for k, v in prof.summary().items()})
    print(U.Benchmark("matmul_1024").warmup(2).iterations(5).run(lambda: a @ a))


if __name__ == "__main__":
    main()
