"""Elastic supervisor: runs a multi-rank job, and when the job stops with a restart marker (a rank was lost between
steps, :mod:`ghost_flow_b200.parallel.fault`), starts it again at the surviving world size from the last sharded
checkpoint.

The job itself does the detecting: survivors notice the missing heartbeat on the host before their next launch, write
``RESTART.json`` (checkpoint directory, failed ranks, old and new world size) and exit with ``EXIT_RESTART``. This module
is the other half: the loop around ``torch.distributed.run``. ``io.load_sharded`` cuts the flat shards of the old
world size again for the new one, so the restarted job continues the same optimizer trajectory.

    python -m ghost_flow_b200.parallel.elastic --nproc 8 --marker-dir run/marker [--divides 64] -- train.py --steps 1000

On a restart the training script finds ``GF_RESUME_FROM`` (checkpoint directory), ``GF_RESTART_COUNT`` and
``GF_PREVIOUS_WORLD`` in its environment. ``--divides B`` restricts the new world size to a divisor of ``B`` (the
global batch). The reference has no failure handling at all (ghostflow-nn/src/distributed.rs has no timeouts, no
heartbeats, no restart).
"""
from __future__ import annotations

import argparse
import os
import subprocess
import sys
from dataclasses import dataclass, field

from . import fault


@dataclass
class ElasticResult:
    returncode: int
    restarts: int
    worlds: list = field(default_factory=list)          # world size of every attempt
    markers: list = field(default_factory=list)         # the restart markers that were acted on


def next_world(marker: dict, divides: int | None = None, min_world: int = 1) -> int:
    """World size of the restarted job: the survivors, or the largest smaller size that divides ``divides``."""
    w = int(marker["new_world"])
    if divides:
        while w > min_world and divides % w:
            w -= 1
    return max(min_world, w)


def run_elastic(script_args, nproc: int, marker_dir, *, max_restarts: int = 3, divides: int | None = None,
                master_addr: str = "127.0.0.1", master_port: int = 29400, env: dict | None = None,
                on_restart=None, timeout: float | None = None, capture: bool = False) -> ElasticResult:
    """Runs ``python -m torch.distributed.run --nproc-per-node nproc script_args...`` until it succeeds, fails without
    a marker, or ``max_restarts`` is used up. ``on_restart(marker, world) -> list`` may return extra script arguments
    for the restarted job (default: none; the environment variables carry the checkpoint directory)."""
    res = ElasticResult(0, 0)
    world = nproc
    extra: list = []
    base_env = dict(os.environ if env is None else env)
    marker_path = os.path.join(os.fspath(marker_dir), fault.RESTART_MARKER)
    while True:
        if os.path.exists(marker_path):
            os.remove(marker_path)                      # a marker from an earlier attempt must not be read again
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
               "--master-addr", master_addr, "--master-port", str(master_port + res.restarts),
               *map(str, script_args), *map(str, extra)]
        r = subprocess.run(cmd, env=base_env, timeout=timeout, capture_output=capture, text=capture)
        res.worlds.append(world)
        res.returncode = r.returncode
        if r.returncode == 0:
            return res
        marker = fault.read_restart_marker(marker_dir)
        if marker is None or res.restarts >= max_restarts:
            return res                                  # a plain failure, or out of attempts: hand the code on
        res.markers.append(marker)
        res.restarts += 1
        world = next_world(marker, divides)
        base_env.update(GF_RESUME_FROM=str(marker["checkpoint_dir"]), GF_RESTART_COUNT=str(res.restarts),
                        GF_PREVIOUS_WORLD=str(marker["old_world"]))
        extra = list(on_restart(marker, world)) if on_restart else []


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--nproc", type=int, required=True)
    ap.add_argument("--marker-dir", required=True)
    ap.add_argument("--max-restarts", type=int, default=3)
    ap.add_argument("--divides", type=int, default=None, help="the new world size must divide this (global batch)")
    ap.add_argument("--master-port", type=int, default=29400)
    ap.add_argument("script", nargs=argparse.REMAINDER, help="-- script.py and its arguments")
    a = ap.parse_args(argv)
    script = a.script[1:] if a.script and a.script[0] == "--" else a.script
    if not script:
        ap.error("no training script given")
    res = run_elastic(script, a.nproc, a.marker_dir, max_restarts=a.max_restarts, divides=a.divides,
                      master_port=a.master_port)
    print(f"[elastic] attempts at world sizes {res.worlds}, {res.restarts} restart(s), exit code {res.returncode}")
    return res.returncode


if __name__ == "__main__":
    raise SystemExit(main())
