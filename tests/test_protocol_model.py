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
