"""The example scripts that run without a GPU finish and print what they promise."""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(args, timeout=300, env=None):
    r = subprocess.run([sys.executable, *args], cwd=ROOT, capture_output=True, text=True, timeout=timeout,
                       env=dict(os.environ, CUDA_VISIBLE_DEVICES="", **(env or {})))
    assert r.returncode == 0, (r.stdout[-1500:], r.stderr[-2500:])
    return r.stdout


def test_basic_usage_example():
    out = _run(["examples/basic_usage.py"])
    assert "trained loss" in out


@pytest.mark.parametrize("world", [1, 2])
def test_mixtral_expert_parallel_example(world):
    args = ["examples/train_mixtral_ep.py"]
    if world > 1:
        args = ["-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
                "--master-port", "29575", *args]
    out = _run(args, env={"MASTER_ADDR": "127.0.0.1", "OMP_NUM_THREADS": "2"})
    losses = [float(line.split("loss")[1].split()[0]) for line in out.splitlines() if line.startswith("step")]
    assert len(losses) == 8 and losses[-1] < losses[0] - 0.5
    assert "experts of layer 0: (4, 256, 64)" in out


def test_step_roofline_budget_is_consistent():
    import json

    out = _run(["benchmarks/step_roofline.py", "--gpus", "8", "--measured-ms", "188.8"])
    b = json.loads(out.strip().splitlines()[-1])
    assert b["model"]["params"] == 6738415616 and b["ideal_step_ms"] == max(b["ideal_compute_ms"], b["ideal_link_ms"])
    gemm = next(r for r in b["parts"] if r["part"].startswith("GEMMs"))
    assert 100 < gemm["ideal_ms"] < 140 and 0.5 < b["fraction_of_ideal"] < 1.0
    one = json.loads(_run(["benchmarks/step_roofline.py", "--gpus", "1"]).strip().splitlines()[-1])
    assert one["ideal_link_ms"] == 0 and one["ideal_compute_ms"] > b["ideal_compute_ms"]      # the whole optimizer on one GPU
