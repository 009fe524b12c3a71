"""The flag protocols of the peer-memory kernels, restated on the host and run with threads as ranks: the complete
rule set never reports a hazard under randomised delays, and taking any single rule away makes the model report
the hazard that rule prevents (so the model would notice a kernel that dropped it)."""
import pytest

from ghost_flow_b200.parallel.protocol_model import ProtocolViolation, Rules, run_moe, run_zero3


@pytest.mark.parametrize("world,regather", [(2, True), (4, True), (8, False), (3, True)])
def test_zero3_flags_order_every_access(world, regather):
    for seed in range(3):
        waits = run_zero3(world=world, units=4, steps=3, seed=seed, regather=regather)
        assert waits > 0


@pytest.mark.parametrize("world", [2, 4, 8])
def test_moe_flags_order_every_access(world):
    for seed in range(3):
        assert run_moe(world=world, calls=5, seed=seed) > 0


def _detects(run, **kw):
    for seed in range(25):
        try:
            run(seed=seed, **kw)
        except ProtocolViolation as e:
            return str(e)
    return None


@pytest.mark.parametrize("rule,needles", [
    ("wait_ready", ("reducer reads",)),
    # a slot rewritten too early shows up as an overwrite under a reader, or as a reducer finding the next unit's data
    ("wait_consumed", ("overwrites grad", "reducer reads")),
    ("wait_version", ("gather reads",))])
def test_zero3_model_notices_a_dropped_rule(rule, needles):
    msg = _detects(run_zero3, world=4, units=4, steps=3, rules=Rules(**{rule: False}), jitter=5e-4)
    assert msg is not None and any(n in msg for n in needles), msg


@pytest.mark.parametrize("rule", ["wait_dispatch", "wait_combine"])
def test_moe_model_notices_a_dropped_rule(rule):
    msg = _detects(run_moe, world=4, calls=6, rules=Rules(**{rule: False}), jitter=5e-4)
    assert msg is not None, rule


# ------------------------------------------------------------------------------------ the C++ model under ThreadSanitizer
import os
import shutil
import subprocess

_SRC = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "ghost_flow_b200", "csrc",
                    "protocol_model.cpp")


@pytest.fixture(scope="module")
def tsan_model(tmp_path_factory):
    if shutil.which("g++") is None:
        pytest.skip("no g++")
    exe = str(tmp_path_factory.mktemp("tsan") / "protocol_model")
    r = subprocess.run(["g++", "-O1", "-g", "-std=c++17", "-fsanitize=thread", _SRC, "-o", exe, "-lpthread"],
                       capture_output=True, text=True)
    if r.returncode != 0:
        pytest.skip("ThreadSanitizer is not available to this compiler: " + r.stderr[-200:])
    return exe


def _tsan(exe, *args):
    env = dict(os.environ, TSAN_OPTIONS="exitcode=66 halt_on_error=1")
    return subprocess.run([exe, *map(str, args)], env=env, capture_output=True, text=True, timeout=300)


@pytest.mark.parametrize("args", [("zero3", 4, 4, 3), ("zero3", 8, 3, 2), ("moe", 4, 6), ("moe", 8, 4)])
def test_flag_protocols_are_race_free_under_thread_sanitizer(tsan_model, args):
    """Flags are std::atomic with the kernels' release / acquire orders, payloads are plain arrays: the sanitizer
    proves that every payload access is ordered by the flags, whatever the timing of the run."""
    r = _tsan(tsan_model, *args)
    assert r.returncode == 0 and "ThreadSanitizer" not in r.stderr and r.stdout.strip() == "ok", r.stderr[-1500:]


@pytest.mark.parametrize("args", [("zero3", 4, 4, 3, "ready"), ("zero3", 4, 4, 3, "consumed"),
                                  ("zero3", 4, 4, 3, "version"), ("moe", 4, 6, "dispatch"), ("moe", 4, 6, "combine")])
def test_thread_sanitizer_reports_a_dropped_rule(tsan_model, args):
    r = _tsan(tsan_model, *args)
    assert r.returncode != 0 and ("data race" in r.stderr or "payload check failed" in r.stderr), (r.returncode, r.stderr[-800:])
