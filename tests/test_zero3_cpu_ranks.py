"""ZeRO-3 engine partitioning logic on CPU ranks (gloo): two ranks with one sequence each must follow the same
loss curve and reach the same weights as one rank with both sequences."""
import os
import subprocess
import sys
import textwrap

import torch

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = textwrap.dedent("""
    import os, sys, json, torch
    import torch.distributed as dist
    sys.path.insert(0, {repo!r})
    from ghost_flow_b200.models.configs import LLaMAConfig
    from ghost_flow_b200.parallel.zero3 import Zero3LlamaEngine, OptimConfig, Comm
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    cfg = LLaMAConfig.llama_tiny()
    eng = Zero3LlamaEngine(cfg, "cpu", optim=OptimConfig(lr=1e-2, max_grad_norm={max_norm}), dtype=torch.float32,
                           seed=7, comm=Comm(), persist_gathered={persist})
    assert eng.persist == {persist}
    g = torch.Generator().manual_seed(11)
    tok = torch.randint(0, cfg.vocab_size, (world, 33), generator=g)
    mine = tok[rank:rank + 1]
    losses = [float(eng.step(mine[:, :-1], mine[:, 1:])) for _ in range(3)]
    w = eng.gather_unit(eng.layers[1], master=True)["w_down"]
    if rank == 0:
        torch.save({{"losses": losses, "w": w}}, {out!r})
    dist.barrier()
    dist.destroy_process_group()
""")


import pytest


@pytest.mark.parametrize("persist", [True, False])
def test_two_cpu_ranks_match_single_rank(tmp_path, persist):
    """Both weight-buffer policies: gathered copies kept from the forward to the backward pass, or two rotating
    buffers with a second gather in the backward pass."""
    from ghost_flow_b200.models.configs import LLaMAConfig
    from ghost_flow_b200.parallel.zero3 import OptimConfig, Zero3LlamaEngine

    out = str(tmp_path / "r0.pt")
    script = tmp_path / "worker.py"
    script.write_text(WORKER.format(repo=REPO, out=out, persist=persist, max_norm=None))
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", OMP_NUM_THREADS="2")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                        "--master-addr", "127.0.0.1", "--master-port", str(29731 + int(persist)), str(script)],
                       env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    got = torch.load(out)
    cfg = LLaMAConfig.llama_tiny()
    eng = Zero3LlamaEngine(cfg, "cpu", optim=OptimConfig(lr=1e-2), dtype=torch.float32, seed=7)
    g = torch.Generator().manual_seed(11)
    tok = torch.randint(0, cfg.vocab_size, (2, 33), generator=g)
    ref = [float(eng.step(tok[:, :-1], tok[:, 1:])) for _ in range(3)]
    for a, b in zip(got["losses"], ref):
        assert abs(a - b) < 1e-4, (got["losses"], ref)
    w = eng.gather_unit(eng.layers[1], master=True)["w_down"]
    assert torch.allclose(got["w"], w, atol=1e-5)


def test_clipped_steps_on_two_cpu_ranks_match_single_rank(tmp_path):
    """The global norm is formed from both ranks' shards (one scalar all-reduce): same clipped curve as one rank."""
    from ghost_flow_b200.models.configs import LLaMAConfig
    from ghost_flow_b200.parallel.zero3 import OptimConfig, Zero3LlamaEngine

    out = str(tmp_path / "r0.pt")
    script = tmp_path / "worker.py"
    script.write_text(WORKER.format(repo=REPO, out=out, persist=True, max_norm=0.1))
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", OMP_NUM_THREADS="2")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                        "--master-addr", "127.0.0.1", "--master-port", "29739", str(script)],
                       env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    got = torch.load(out)
    cfg = LLaMAConfig.llama_tiny()
    eng = Zero3LlamaEngine(cfg, "cpu", optim=OptimConfig(lr=1e-2, max_grad_norm=0.1), dtype=torch.float32, seed=7)
    g = torch.Generator().manual_seed(11)
    tok = torch.randint(0, cfg.vocab_size, (2, 33), generator=g)
    ref = [float(eng.step(tok[:, :-1], tok[:, 1:])) for _ in range(3)]
    assert eng.last_stats["clip_coef"] < 1.0
    for a, b in zip(got["losses"], ref):
        assert abs(a - b) < 1e-4, (got["losses"], ref)
    assert torch.allclose(got["w"], eng.gather_unit(eng.layers[1], master=True)["w_down"], atol=1e-5)


def test_global_norm_clipping_and_skipped_step_single_rank():
    """max_grad_norm: the update is deferred until the global norm is known; the norm equals the norm of the
    gradients an unclipped engine would have applied, the clip coefficient scales the update, and a non-finite
    norm leaves weights, moments and the step count untouched."""
    from ghost_flow_b200.models.configs import LLaMAConfig
    from ghost_flow_b200.parallel.zero3 import OptimConfig, Zero3LlamaEngine

    cfg = LLaMAConfig.llama_tiny()
    g = torch.Generator().manual_seed(11)
    tok = torch.randint(0, cfg.vocab_size, (2, 33), generator=g)
    free = Zero3LlamaEngine(cfg, "cpu", optim=OptimConfig(lr=1e-2), dtype=torch.float32, seed=7)
    big = Zero3LlamaEngine(cfg, "cpu", optim=OptimConfig(lr=1e-2, max_grad_norm=1e9), dtype=torch.float32, seed=7)
    tight = Zero3LlamaEngine(cfg, "cpu", optim=OptimConfig(lr=1e-2, max_grad_norm=0.05), dtype=torch.float32, seed=7)
    l0 = [float(free.step(tok[:, :-1], tok[:, 1:])) for _ in range(3)]
    l1 = [float(big.step(tok[:, :-1], tok[:, 1:])) for _ in range(3)]
    assert all(abs(a - b) < 1e-6 for a, b in zip(l0, l1))             # a bound never reached changes nothing
    assert big.last_stats["clip_coef"] == 1.0 and big.last_stats["grad_norm"] > 0.05
    w_before = tight.layers[0].master.clone()
    tight.step(tok[:, :-1], tok[:, 1:])
    st = tight.last_stats
    assert not st["skipped"] and abs(st["clip_coef"] - 0.05 / (st["grad_norm"] + 1e-6)) < 1e-9
    # first AdamW step: |update| = lr * g / (|g| + eps) whatever the scale, so compare the moments instead
    ref = Zero3LlamaEngine(cfg, "cpu", optim=OptimConfig(lr=1e-2, max_grad_norm=1e9), dtype=torch.float32, seed=7)
    ref.step(tok[:, :-1], tok[:, 1:])
    assert torch.allclose(tight.layers[0].m, ref.layers[0].m * st["clip_coef"], rtol=1e-5, atol=1e-12)
    assert not torch.equal(tight.layers[0].master, w_before)
    # a poisoned weight makes the loss and every gradient non-finite: the step must be skipped
    tight.layers[1].master[5] = float("inf")
    tight.layers[1].shard.copy_(tight.layers[1].master)
    snap = (tight.layers[0].master.clone(), tight.layers[0].m.clone(), tight.step_count)
    tight.step(tok[:, :-1], tok[:, 1:])
    assert tight.last_stats["skipped"] and tight.skipped_steps == 1
    assert tight.step_count == snap[2]
    assert torch.equal(tight.layers[0].master, snap[0]) and torch.equal(tight.layers[0].m, snap[1])


def test_activation_recompute_gives_the_same_step():
    """Keeping only the layer inputs and re-running each layer's forward pass in the backward pass changes nothing in
    the numbers (fp32 on CPU: bit-identical)."""
    from ghost_flow_b200.models.configs import LLaMAConfig
    from ghost_flow_b200.parallel.zero3 import OptimConfig, Zero3LlamaEngine

    cfg = LLaMAConfig(vocab_size=128, hidden_size=32, intermediate_size=64, num_hidden_layers=3,
                      num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=32)
    g = torch.Generator().manual_seed(0)
    tok = torch.randint(0, 128, (2, 17), generator=g)
    runs = []
    for rec in (False, True):
        eng = Zero3LlamaEngine(cfg, "cpu", optim=OptimConfig(lr=1e-2), dtype=torch.float32, seed=7,
                               recompute_activations=rec)
        losses = [float(eng.step(tok[:, :-1], tok[:, 1:])) for _ in range(3)]
        runs.append((losses, eng.gather_unit(eng.layers[1], master=True)["wqkv"].clone()))
    assert runs[0][0] == runs[1][0] and torch.equal(runs[0][1], runs[1][1])


@pytest.mark.parametrize("clip", [None, 0.05])
def test_gradient_accumulation_equals_one_large_batch(clip):
    """Two micro-batches through accumulate() + step() against one step on both at once (the loss is a token mean
    and the micro-batches have equal size, so the accumulated mean gradient is the large batch's gradient)."""
    from ghost_flow_b200.models.configs import LLaMAConfig
    from ghost_flow_b200.parallel.zero3 import OptimConfig, Zero3LlamaEngine

    cfg = LLaMAConfig(vocab_size=128, hidden_size=32, intermediate_size=64, num_hidden_layers=2,
                      num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=32)
    g = torch.Generator().manual_seed(0)
    tok = torch.randint(0, 128, (4, 17), generator=g)
    mk = lambda: Zero3LlamaEngine(cfg, "cpu", optim=OptimConfig(lr=1e-2, max_grad_norm=clip), dtype=torch.float32,  # noqa: E731
                                  seed=7)
    big, acc = mk(), mk()
    for _ in range(3):
        lb = float(big.step(tok[:, :-1], tok[:, 1:]))
        l1 = float(acc.accumulate(tok[:2, :-1], tok[:2, 1:]))
        l2 = float(acc.step(tok[2:, :-1], tok[2:, 1:]))
        assert abs(lb - 0.5 * (l1 + l2)) < 1e-5
        assert acc.last_stats["micro_batches"] == 2
        if clip is not None:
            assert abs(acc.last_stats["grad_norm"] - big.last_stats["grad_norm"]) < 1e-4 * big.last_stats["grad_norm"]
            assert abs(acc.last_stats["clip_coef"] - big.last_stats["clip_coef"]) < 1e-4
    wa = acc.gather_unit(acc.layers[1], master=True)["w_down"]
    wb = big.gather_unit(big.layers[1], master=True)["w_down"]
    assert ((wa - wb).norm() / wb.norm()).item() < 1e-5
    assert acc.step_count == big.step_count == 3


ACC_WORKER = textwrap.dedent("""
    import os, sys, torch
    import torch.distributed as dist
    sys.path.insert(0, {repo!r})
    from ghost_flow_b200.models.configs import LLaMAConfig
    from ghost_flow_b200.parallel.zero3 import Zero3LlamaEngine, OptimConfig, Comm
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    cfg = LLaMAConfig.llama_tiny()
    eng = Zero3LlamaEngine(cfg, "cpu", optim=OptimConfig(lr=1e-2, max_grad_norm=0.1), dtype=torch.float32, seed=7,
                           comm=Comm(), recompute_activations=True)
    g = torch.Generator().manual_seed(11)
    tok = torch.randint(0, cfg.vocab_size, (2 * world, 33), generator=g)
    a, b = tok[rank:rank + 1], tok[world + rank:world + rank + 1]      # two micro-batches of one sequence per rank
    losses = []
    for _ in range(3):
        l1 = float(eng.accumulate(a[:, :-1], a[:, 1:]))
        l2 = float(eng.step(b[:, :-1], b[:, 1:]))
        losses.append(0.5 * (l1 + l2))
    w = eng.gather_unit(eng.layers[1], master=True)["w_down"]
    if rank == 0:
        torch.save({{"losses": losses, "w": w, "stats": dict(eng.last_stats)}}, {out!r})
    dist.barrier()
    dist.destroy_process_group()
""")


def test_accumulation_clipping_and_recompute_on_two_cpu_ranks_match_one_large_batch(tmp_path):
    """Everything at once on gloo ranks: two micro-batches per step and rank, global-norm clipping of the accumulated
    gradient, activations recomputed in the backward pass; against one rank stepping on all four sequences."""
    from ghost_flow_b200.models.configs import LLaMAConfig
    from ghost_flow_b200.parallel.zero3 import OptimConfig, Zero3LlamaEngine

    out = str(tmp_path / "acc.pt")
    script = tmp_path / "worker.py"
    script.write_text(ACC_WORKER.format(repo=REPO, out=out))
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", OMP_NUM_THREADS="2")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                        "--master-addr", "127.0.0.1", "--master-port", "29737", str(script)],
                       env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    got = torch.load(out)
    cfg = LLaMAConfig.llama_tiny()
    eng = Zero3LlamaEngine(cfg, "cpu", optim=OptimConfig(lr=1e-2, max_grad_norm=0.1), dtype=torch.float32, seed=7)
    g = torch.Generator().manual_seed(11)
    tok = torch.randint(0, cfg.vocab_size, (4, 33), generator=g)
    ref = [float(eng.step(tok[:, :-1], tok[:, 1:])) for _ in range(3)]
    for a, b in zip(got["losses"], ref):
        assert abs(a - b) < 1e-4, (got["losses"], ref)
    assert got["stats"]["micro_batches"] == 2 and got["stats"]["clip_coef"] < 1.0
    assert abs(got["stats"]["grad_norm"] - eng.last_stats["grad_norm"]) < 1e-3 * eng.last_stats["grad_norm"]
    w = eng.gather_unit(eng.layers[1], master=True)["w_down"]
    assert torch.allclose(got["w"], w, atol=2e-5)
