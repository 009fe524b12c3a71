"""Multi-GPU ZeRO-3: this package's peer-memory collectives (all-gather pull, reduce-scatter fused with AdamW)
against the NCCL path and against a single GPU holding the whole batch."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def _need(n):
    if torch.cuda.device_count() < n:
        pytest.skip(f"needs {n} GPUs")


def _run(kind, out, n, steps=4, port=29741, **extra_env):
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", **extra_env)
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
                        "--master-addr", "127.0.0.1", "--master-port", str(port),
                        os.path.join(HERE, "_multi_gpu_worker.py"), kind, out, str(steps)],
                       env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, (r.stdout[-1500:], r.stderr[-3000:])
    return torch.load(out)


@pytest.mark.parametrize("world", [2, 4, 8])
def test_fused_collectives_match_nccl_and_single_gpu(tmp_path, world):
    """Every world size exercises other code: two batches of four peer loads in the fused reducer only at 8 ranks,
    the second batch half full at more than 4."""
    _need(world)
    from ghost_flow_b200.models.configs import LLaMAConfig
    from ghost_flow_b200.parallel.zero3 import OptimConfig, Zero3LlamaEngine

    fused = _run("fused", str(tmp_path / "f.pt"), world, port=29741)
    nccl = _run("nccl", str(tmp_path / "n.pt"), world, port=29743)
    assert fused["fused"], "the peer-memory path was not taken"
    cfg = LLaMAConfig(vocab_size=2048, hidden_size=512, intermediate_size=1024, num_hidden_layers=4,
                      num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=512)
    eng = Zero3LlamaEngine(cfg, "cuda", optim=OptimConfig(lr=2e-3), seed=5)
    g = torch.Generator().manual_seed(99)
    tok = torch.randint(0, cfg.vocab_size, (world, 257), generator=g).cuda()
    single = [float(eng.step(tok[:, :-1], tok[:, 1:])) for _ in range(4)]
    for a, b, c in zip(fused["losses"], nccl["losses"], single):
        assert abs(a - b) < 2e-2 and abs(a - c) < 3e-2, (fused["losses"], nccl["losses"], single)
    w1 = eng.gather_unit(eng.layers[2], master=True)["w_gate_up"].cpu()
    assert (fused["w"] - nccl["w"]).norm() / nccl["w"].norm() < 1e-2
    assert (fused["w"] - w1).norm() / w1.norm() < 1e-2


def test_fused_path_resumes_from_a_sharded_checkpoint(tmp_path):
    """Save after two steps, load into a new engine with a new communicator (zeroed flags, step counter = 2) and
    continue: the loss curve must be the uninterrupted one. Also with the rotating (non-persistent) weight buffers."""
    _need(2)
    plain = _run("fused", str(tmp_path / "f.pt"), 2, port=29745)
    resumed = _run("fused_resume", str(tmp_path / "r.pt"), 2, port=29747)
    rotating = _run("fused_resume_nopersist", str(tmp_path / "q.pt"), 2, port=29749)
    # independent bf16 runs drift apart by a few 1e-3 in the loss within four AdamW steps (see below); a resume
    # on stale or zero weights would be off by whole units
    for a, b, c in zip(plain["losses"], resumed["losses"], rotating["losses"]):
        assert abs(a - b) < 1e-2 and abs(a - c) < 1e-2, (plain["losses"], resumed["losses"], rotating["losses"])
    # two runs of the same job already differ in the last bits (the attention backward adds dQ tiles in arrival
    # order) and AdamW turns that into differences of a few 1e-3 after four steps at this learning rate
    rel = ((plain["w"] - resumed["w"]).norm() / plain["w"].norm()).item()
    assert rel < 1e-2, rel


def test_clipped_steps_fused_reduce_only_matches_nccl(tmp_path):
    """Gradient clipping on the peer-memory path: the reducer runs in its reduce-only mode (fp32 shard + sum of
    squares), AdamW follows once the global norm is known, version flags are published after it."""
    _need(2)
    fused = _run("fused_clip", str(tmp_path / "f.pt"), 2, port=29765)
    nccl = _run("nccl_clip", str(tmp_path / "n.pt"), 2, port=29767)
    assert fused["fused"] and fused["stats"]["clip_coef"] < 1.0 and not fused["stats"]["skipped"]
    assert abs(fused["stats"]["grad_norm"] - nccl["stats"]["grad_norm"]) < 2e-2 * nccl["stats"]["grad_norm"]
    for a, b in zip(fused["losses"], nccl["losses"]):
        assert abs(a - b) < 2e-2, (fused["losses"], nccl["losses"])
    assert (fused["w"] - nccl["w"]).norm() / nccl["w"].norm() < 1e-2


def test_fused_tensor_parallel_kernels_match_nccl(tmp_path):
    """all-gather + GEMM and GEMM + reduce-scatter as single kernels against NCCL followed / preceded by the GEMM."""
    _need(2)
    out = str(tmp_path / "tp.pt")
    env = dict(os.environ, MASTER_ADDR="127.0.0.1")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                        "--master-addr", "127.0.0.1", "--master-port", "29751",
                        os.path.join(HERE, "_tp_worker.py"), out], env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, (r.stdout[-1500:], r.stderr[-3000:])
    res = torch.load(out)
    assert res and all(v < 1.5e-2 for v in res.values()), res


def test_expert_parallel_moe_matches_dense_reference(tmp_path):
    """Experts sharded over 2 GPUs: dispatch / combine over peer memory and grouped GEMMs against the dense oracle."""
    _need(2)
    out = str(tmp_path / "ep.pt")
    env = dict(os.environ, MASTER_ADDR="127.0.0.1")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                        "--master-addr", "127.0.0.1", "--master-port", "29753",
                        os.path.join(HERE, "_ep_worker.py"), out], env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, (r.stdout[-1500:], r.stderr[-3000:])
    res = torch.load(out)
    assert res and all(v < 5e-2 for v in res.values()), res


def test_context_parallel_attention_matches_single_gpu(tmp_path):
    """Ring attention (K/V and dK/dV travelling over NCCL p2p) and Ulysses against FlashAttention on the full sequence."""
    _need(2)
    out = str(tmp_path / "cp.pt")
    env = dict(os.environ, MASTER_ADDR="127.0.0.1")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                        "--master-addr", "127.0.0.1", "--master-port", "29755",
                        os.path.join(HERE, "_cp_worker.py"), out], env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, (r.stdout[-1500:], r.stderr[-3000:])
    res = torch.load(out)
    assert res and all(v < 3e-2 for v in res.values()), res


def test_tensor_parallel_inference_matches_single_gpu(tmp_path):
    """Prefill + greedy decode with heads and MLP columns sharded over 2 GPUs (fused, NCCL and fp8 linears)."""
    _need(2)
    out = str(tmp_path / "tpinf.pt")
    env = dict(os.environ, MASTER_ADDR="127.0.0.1")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                        "--master-addr", "127.0.0.1", "--master-port", "29757",
                        os.path.join(HERE, "_tpinf_worker.py"), out], env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, (r.stdout[-1500:], r.stderr[-3000:])
    res = torch.load(out)
    for mode in ("fused", "nccl"):
        assert res[f"{mode}_logit_rel"] < 3e-2 and res[f"{mode}_first_token_agreement"] == 1.0, res
        assert res[f"{mode}_token_agreement"] >= 0.75, res
    assert res["fp8_logit_rel"] < 0.15, res


def test_zero2_reduce_scatter_fused_with_adamw_matches_nccl(tmp_path):
    """Generic ZeRO-2 optimizer: per bucket one peer-memory kernel (gradient reduce-scatter + AdamW) and a pull
    all-gather, against NCCL reduce-scatter / all-gather around the flat AdamW kernel."""
    _need(2)
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", NCCL_NVLS_ENABLE="0")   # the NCCL arm needs no in-switch reduction
    res = {}
    for kind, port in (("fused", 29761), ("nccl", 29763), ("fused_late", 29779), ("fused_graph", 29781),
                       ("nccl_graph", 29783)):
        out = str(tmp_path / f"z2_{kind}.pt")
        r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                            "--master-addr", "127.0.0.1", "--master-port", str(port),
                            os.path.join(HERE, "_zero2_worker.py"), kind, out, "6"],
                           env=env, capture_output=True, text=True, timeout=600)
        assert r.returncode == 0, (r.stdout[-1500:], r.stderr[-3000:])
        res[kind] = torch.load(out)
    assert res["fused"]["fused"] and not res["nccl"]["fused"] and res["fused"]["buckets"] >= 2
    # default: launched from gradient hooks under the backward pass; _late: after it; _graph: the whole step (hooks,
    # side stream, flag values and Adam step number from a device counter) replayed from one CUDA graph
    assert res["fused"]["overlap"] and not res["fused_late"]["overlap"] and res["fused_graph"]["graph"]
    for other in ("nccl", "fused_late", "fused_graph", "nccl_graph"):
        for a, b in zip(res["fused"]["losses"], res[other]["losses"]):
            assert abs(a - b) < 3e-2, (other, res["fused"]["losses"], res[other]["losses"])
        assert (res["fused"]["w"] - res[other]["w"]).norm() / res["fused"]["w"].norm() < 2e-2, other
    assert res["fused"]["losses"][-1] < res["fused"]["losses"][0]
    assert (res["fused"]["w"] - res["nccl"]["w"]).norm() / res["nccl"]["w"].norm() < 2e-2


@pytest.mark.parametrize("world", [1, 2])
def test_mixtral_expert_parallel_engine_matches_cpu_fp32(tmp_path, world):
    """Mixtral training: attention parameters under ZeRO-3 (peer-memory collectives), experts owned by the ranks
    (dispatch / combine kernels over peer memory, grouped GEMMs, local AdamW), router gradient all-reduced; against
    the same engine on one CPU rank in fp32 on the whole batch."""
    _need(world)
    sys.path.insert(0, HERE)
    import _mixtral_worker as mw
    from ghost_flow_b200.parallel.mixtral import MixtralEngine
    from ghost_flow_b200.parallel.zero3 import OptimConfig

    out = str(tmp_path / "mx.pt")
    env = dict(os.environ, MASTER_ADDR="127.0.0.1")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
                        "--master-addr", "127.0.0.1", "--master-port", "29771",
                        os.path.join(HERE, "_mixtral_worker.py"), "fused", out, "4"],
                       env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, (r.stdout[-1500:], r.stderr[-3000:])
    got = torch.load(out)
    assert got["fused"] == (world > 1)
    cfg = mw.config()
    tok = mw.batch(world)
    # a small learning rate: the first Adam steps move every weight by lr whatever its gradient's size, so elements
    # whose bf16 gradient has the other sign than the fp32 one separate the two runs in proportion to lr
    ref = MixtralEngine(cfg, "cpu", tokens_per_rank=tok.shape[0] * 256, optim=OptimConfig(lr=5e-4, weight_decay=0.0),
                        dtype=torch.float32, seed=5)
    ref.load_full_state(got["init"])     # the dense weights are drawn on the device; the experts on the host
    want = [float(ref.step(tok[:, :-1], tok[:, 1:])) for _ in range(4)]
    assert want[-1] < want[0]
    assert abs(got["losses"][0] - want[0]) < 5e-3 and abs(got["losses"][1] - want[1]) < 1e-2, (got["losses"], want)
    # later steps drift: a token whose two best experts are nearly tied goes to another expert in bf16
    for i, (a, b) in enumerate(zip(got["losses"], want)):
        assert abs(a - b) < (2e-2 if i < 3 else 1e-1), (got["losses"], want)
    e = ref.experts[1]
    for name, w in (("w13_e0", e.master["w13"][0]), ("w2_e0", e.master["w2"][0]), ("gate", e.master["gate"])):
        rel = ((got[name] - w).norm() / w.norm()).item()
        # the router sees the smallest gradients, and at world > 1 its load-balancing term uses each rank's own token
        # fractions where the one-rank run uses the whole batch's
        assert rel < (5e-2 if name == "gate" else 3e-2), (name, rel)
    wq = ref.gather_unit(ref.layers[1], master=True)["wqkv"]
    assert ((got["wqkv"] - wq).norm() / wq.norm()).item() < 2e-2


def test_pipeline_1f1b_over_nccl_matches_whole_model(tmp_path):
    """Two stages on two GPUs, four micro-batches, activations and their gradients over NCCL send/recv (each exchange
    with a neighbour is one grouped batch): loss and every stage's gradients against the whole model on one GPU."""
    _need(2)
    out = str(tmp_path / "pp.pt")
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                        "--master-addr", "127.0.0.1", "--master-port", "29773",
                        os.path.join(HERE, "_pp_worker.py"), out], env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, (r.stdout[-1500:], r.stderr[-3000:])
    res = [torch.load(f"{out}.{i}") for i in range(2)]
    for d in res:
        assert d["n_grads"] > 0 and d["grad_rel"] < 2e-2, res
    assert res[1]["loss_err"] < 1e-2, res


def test_in_switch_reduction_variant_of_the_fused_reducer_matches_peer_loads(tmp_path):
    """``GF_MULTIMEM=1``: the reducer reads the gradient with ``multimem.ld_reduce`` (one load, summed inside the
    NVSwitch) instead of one load per peer. Same job as the default path, same losses and weights."""
    _need(2)
    plain = _run("fused", str(tmp_path / "p.pt"), 2, port=29775)
    mm = _run("fused", str(tmp_path / "m.pt"), 2, port=29777, GF_MULTIMEM="1")
    if not mm["multimem"]:
        pytest.skip("no multicast mapping on this system")
    assert mm["fused"] and not plain["multimem"]
    for a, b in zip(plain["losses"], mm["losses"]):
        assert abs(a - b) < 1e-2, (plain["losses"], mm["losses"])
    assert (plain["w"] - mm["w"]).norm() / plain["w"].norm() < 1e-2
