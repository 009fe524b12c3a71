"""Sharded checkpoints of the ZeRO-3 engine on CPU ranks (gloo): bitwise resume at the same world size, resume at
another world size (the flat shards are cut again), a consolidated checkpoint with the optimizer moments, and an
elastic restart after a host-injected rank loss. The reference keeps params / optimizer state / epoch / loss / extra
in its checkpoint (ghostflow-nn/src/serialization.rs:12-37,144-162,268-284) but has no partitioned state and never
resumes a run."""
import json
import os
import subprocess
import sys

import torch

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
WORKER = os.path.join(REPO, "tests", "_resume_worker.py")
_PORT = [29750]


def _launch(world, *args, expect=0, timeout=300):
    _PORT[0] += 1
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", OMP_NUM_THREADS="1")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
                        "--master-addr", "127.0.0.1", "--master-port", str(_PORT[0]), WORKER, *map(str, args)],
                       env=env, capture_output=True, text=True, timeout=timeout)
    if expect == 0:
        assert r.returncode == 0, r.stderr[-3000:]
    else:
        assert r.returncode != 0, "the run was expected to stop"
    return r


def test_resume_at_same_world_size_is_bitwise_equal_to_uninterrupted_run(tmp_path):
    ck = tmp_path / "ck"
    _launch(2, "--steps", 6, "--out", tmp_path / "full.pt")
    _launch(2, "--steps", 3, "--save", ck, "--out", tmp_path / "a.pt")
    _launch(2, "--steps", 3, "--load", ck, "--out", tmp_path / "b.pt")
    full, a, b = (torch.load(tmp_path / n) for n in ("full.pt", "a.pt", "b.pt"))
    assert a["losses"] + b["losses"] == full["losses"]          # bitwise: same floats
    assert a["lrs"] + b["lrs"] == full["lrs"]                   # the scheduler continued where it stopped
    assert b["step"] == 6
    assert torch.equal(b["w"], full["w"]) and torch.equal(b["m"], full["m"])
    files = sorted(os.listdir(ck))
    assert files == ["shard_00000_of_00002.gfcp", "shard_00001_of_00002.gfcp"]


def test_resume_at_another_world_size_recuts_the_shards(tmp_path):
    ck = tmp_path / "ck"
    _launch(2, "--steps", 5, "--out", tmp_path / "full.pt")
    _launch(2, "--steps", 3, "--save", ck, "--out", tmp_path / "a.pt")
    full = torch.load(tmp_path / "full.pt")
    for world in (1, 4):
        out = tmp_path / f"w{world}.pt"
        _launch(world, "--steps", 2, "--load", ck, "--out", out)
        got = torch.load(out)
        for x, y in zip(got["losses"], full["losses"][3:]):
            assert abs(x - y) < 1e-5, (world, got["losses"], full["losses"])
        assert torch.allclose(got["w"], full["w"], atol=1e-6)
        assert torch.allclose(got["m"], full["m"], atol=1e-7)   # the Adam moments travelled with the weights


def test_consolidated_checkpoint_carries_the_moments(tmp_path):
    """Single process: consolidate(with_optimizer=True) -> a fresh engine -> load_consolidated continues exactly."""
    from ghost_flow_b200 import io as gio
    from ghost_flow_b200.models.configs import LLaMAConfig
    from ghost_flow_b200.parallel.zero3 import OptimConfig, Zero3LlamaEngine

    cfg = LLaMAConfig.llama_tiny()
    g = torch.Generator().manual_seed(3)
    tok = torch.randint(0, cfg.vocab_size, (2, 33), generator=g)

    def make():
        return Zero3LlamaEngine(cfg, "cpu", optim=OptimConfig(lr=1e-2), dtype=torch.float32, seed=7)

    ref = make()
    ref_losses = [float(ref.step(tok[:, :-1], tok[:, 1:])) for _ in range(4)]
    a = make()
    la = [float(a.step(tok[:, :-1], tok[:, 1:])) for _ in range(2)]
    path = tmp_path / "full.gfcp"
    gio.consolidate(a, path, with_optimizer=True)
    b = Zero3LlamaEngine(cfg, "cpu", optim=OptimConfig(lr=1e-2), dtype=torch.float32, seed=99)   # other weights
    gio.load_consolidated(b, path)
    lb = [float(b.step(tok[:, :-1], tok[:, 1:])) for _ in range(2)]
    assert la + lb == ref_losses
    # the plain state-dict form still works and holds only weights
    gio.consolidate(a, tmp_path / "w.gf")
    sd = gio.load_state_dict(tmp_path / "w.gf")
    assert set(sd) == set(a.state_dict())


def test_rng_scaler_and_position_round_trip_through_extra(tmp_path):
    from ghost_flow_b200 import io as gio
    from ghost_flow_b200.nn.mixed_precision import GradScaler, MixedPrecisionConfig

    scaler = GradScaler(MixedPrecisionConfig.fp16())
    scaler.scale = 512.0 if hasattr(scaler, "scale") else None
    torch.manual_seed(5)
    torch.rand(3)
    ex = gio.training_state_extra(scaler=scaler, data_position=17)
    expect = torch.rand(4)
    gio.save_checkpoint(gio.Checkpoint({"w": torch.ones(2)}, None, 1, 0.5, "m", extra=ex), tmp_path / "c.gfcp")
    back = gio.load_checkpoint(tmp_path / "c.gfcp")
    torch.manual_seed(123)
    s2 = GradScaler(MixedPrecisionConfig.fp16())
    got = gio.restore_training_state(back.extra, scaler=s2)
    assert got["data_position"] == 17
    assert torch.equal(torch.rand(4), expect)                  # the generator continues where it was saved
    assert s2.state_dict() == scaler.state_dict()


def test_rank_loss_between_steps_restarts_at_smaller_world(tmp_path):
    """Four ranks save after step 2; rank 3 leaves before step 4 (host-side injection). The survivors notice on the
    host before their next launch, write the restart marker and stop; the job restarts at a smaller world size from
    the last sharded checkpoint and the loss curve continues as if nothing had happened."""
    ck, mk = tmp_path / "ck", tmp_path / "marker"
    _launch(2, "--steps", 5, "--out", tmp_path / "full.pt")
    _launch(4, "--steps", 6, "--save", ck, "--save-at", 2, "--die-rank", 3, "--die-step", 3, "--marker-dir", mk,
            "--out", tmp_path / "broken", expect=1)
    from ghost_flow_b200.parallel import fault

    marker = fault.read_restart_marker(mk)
    assert marker is not None and marker["failed_ranks"] == [3] and marker["old_world"] == 4
    assert marker["new_world"] == 3 and marker["checkpoint_dir"] == str(ck)
    partial = json.load(open(str(tmp_path / "broken") + ".partial.json"))
    assert len(partial["losses"]) == 3 and partial["exit"] == fault.EXIT_RESTART
    # the global batch of 4 sequences does not divide by 3 ranks, so the restart takes the next smaller size that does
    new_world = max(w for w in range(1, marker["new_world"] + 1) if 4 % w == 0)
    _launch(new_world, "--steps", 3, "--load", marker["checkpoint_dir"], "--out", tmp_path / "resumed.pt")
    full, got = torch.load(tmp_path / "full.pt"), torch.load(tmp_path / "resumed.pt")
    assert got["step"] == 5
    for x, y in zip(got["losses"], full["losses"][2:]):
        assert abs(x - y) < 1e-5, (got["losses"], full["losses"])
    for x, y in zip(partial["losses"], full["losses"]):
        assert abs(x - y) < 1e-5


def test_elastic_supervisor_restarts_the_job_at_the_surviving_world_size(tmp_path):
    """The loop around the launcher: the job loses rank 3 between steps, the survivors write the marker and exit, the
    supervisor starts the job again at the largest world size that still divides the global batch, from the sharded
    checkpoint; the continued loss curve is the uninterrupted one."""
    from ghost_flow_b200.parallel import elastic, fault

    ck, mk = tmp_path / "ck", tmp_path / "marker"
    _launch(2, "--steps", 5, "--out", tmp_path / "full.pt")
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", OMP_NUM_THREADS="1")
    res = elastic.run_elastic(
        [WORKER, "--steps", 6, "--save", ck, "--save-at", 2, "--die-rank", 3, "--die-step", 3, "--marker-dir", mk,
         "--out", tmp_path / "broken"],
        nproc=4, marker_dir=mk, divides=4, master_port=29790, env=env, capture=True, timeout=600,
        on_restart=lambda marker, world: ["--steps", 3, "--load", marker["checkpoint_dir"], "--die-rank", -1,
                                          "--save", "", "--out", tmp_path / "resumed.pt"])
    assert res.returncode == 0 and res.restarts == 1 and res.worlds == [4, 2], res
    assert res.markers[0]["failed_ranks"] == [3] and res.markers[0]["old_world"] == 4
    assert elastic.next_world({"new_world": 7}, divides=64) == 4 and elastic.next_world({"new_world": 7}) == 7
    full, got = torch.load(tmp_path / "full.pt"), torch.load(tmp_path / "resumed.pt")
    assert got["step"] == 5
    for x, y in zip(got["losses"], full["losses"][2:]):
        assert abs(x - y) < 1e-5, (got["losses"], full["losses"])
    # a job that fails without a marker is not restarted
    plain = elastic.run_elastic([WORKER, "--no-such-flag"], nproc=1, marker_dir=tmp_path / "none", master_port=29795,
                                env=env, capture=True, timeout=300)
    assert plain.returncode != 0 and plain.restarts == 0 and plain.worlds == [1]
    assert fault.read_restart_marker(tmp_path / "none") is None
