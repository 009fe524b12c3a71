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
