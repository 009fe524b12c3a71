"""Small public types of the reference that other code passes around: checkpoint object and metadata, parameter
partition records, the scheduler base, allocation statistics, difficulty metrics, replay-buffer experiences."""
import torch

import ghost_flow_b200 as gf
from ghost_flow_b200 import io as gio
from ghost_flow_b200.models import Experience, ReplayBuffer
from ghost_flow_b200.nn import CurriculumConfig, DifficultyMetric, DifficultyScorer
from ghost_flow_b200.optim import SGD, LRScheduler, StepLR
from ghost_flow_b200.parallel.distributed import ParameterPartition, ZeRoConfig, ZeRoOptimizer
from ghost_flow_b200.utils import AllocationStats, TrackedAllocator


def test_model_checkpoint_round_trip(tmp_path):
    params = {"fc.weight": torch.randn(4, 3), "fc.bias": torch.randn(4)}
    ck = gio.ModelCheckpoint(params, gio.ModelMetadata(name="mlp", epoch=7, loss=0.25, extra={"lr": "0.01"}))
    ck.with_optimizer_state({"fc.weight.exp_avg": torch.ones(12)})
    path = tmp_path / "m.gfcp"
    ck.save(path)
    back = gio.ModelCheckpoint.load(path)
    assert back.metadata.name == "mlp" and back.metadata.epoch == 7 and abs(back.metadata.loss - 0.25) < 1e-7
    assert back.metadata.extra["lr"] == "0.01"
    assert torch.equal(back.parameters["fc.weight"], params["fc.weight"])
    assert torch.equal(back.optimizer_state["fc.weight.exp_avg"], torch.ones(12))


def test_parameter_partitions_cover_every_element_once():
    ps = [torch.nn.Parameter(torch.randn(10, 7)), torch.nn.Parameter(torch.randn(33)),
          torch.nn.Parameter(torch.randn(5, 5))]
    opt = ZeRoOptimizer(ps, ZeRoConfig(bucket_size=80))
    parts = opt.parameter_partitions(["a", "b", "c"])
    assert [p.name for p in parts] == ["a", "b", "c"] and all(isinstance(p, ParameterPartition) for p in parts)
    assert parts[0].shape == (10, 7) and parts[0].end_idx - parts[0].start_idx == 70
    assert parts[1].bucket == 1 and parts[1].start_idx == 0          # 70 + 33 > 80: a new bucket
    assert all(p.owner_rank == 0 and p.owners == (0,) for p in parts)  # one rank owns everything


def test_scheduler_base_and_allocation_stats():
    w = torch.nn.Parameter(torch.zeros(2))
    sched = StepLR(SGD([w], lr=0.1), step_size=2, gamma=0.5)
    assert isinstance(sched, LRScheduler)
    for _ in range(2):
        sched.step()
    assert abs(sched.get_lr() - 0.05) < 1e-9
    alloc = TrackedAllocator()
    a = alloc.allocate((256, 1024))
    b = alloc.allocate((512, 1024))
    alloc.free(a)
    st = alloc.allocation_stats()
    assert isinstance(st, AllocationStats) and st.allocations == 2 and st.deallocations == 1
    assert st.peak_mb() == 3.0 and st.current_mb() == 2.0 and st.total_mb() == 3.0
    del b


def test_difficulty_metric_and_experience():
    assert CurriculumConfig(metric="loss").difficulty_metric is DifficultyMetric.Loss
    conf = DifficultyScorer(DifficultyMetric.Confidence).score([0.9, 0.5, 0.1])
    assert conf[0] < conf[1] < conf[2]                    # the confident sample is the easy one
    custom = DifficultyScorer(DifficultyMetric.Custom, fn=len).score(["ab", "abcd", "a"])
    assert custom.argmax() == 1
    buf = ReplayBuffer(4)
    buf.push(Experience(torch.zeros(3), 1, 0.5, torch.ones(3), False))
    buf.push(torch.ones(3), 2, -1.0, torch.zeros(3), True)
    s, a, r, s2, d = buf.sample(2)
    assert s.shape == (2, 3) and sorted(a.tolist()) == [1, 2] and gf is not None


def test_small_nn_types():
    from ghost_flow_b200 import nn
    from ghost_flow_b200.models import AggregatorType, GraphSAGELayer
    from ghost_flow_b200.utils import Profiler, ProfileRecord, ProfileSummary

    # QLoRA base weights in the three storage formats: the finer the code book, the smaller the error
    torch.manual_seed(0)
    errs = {}
    for qt in (nn.QuantType.FP4, nn.QuantType.NF4, nn.QuantType.INT8):
        lin = nn.QLoRALinear(64, 32, nn.QLoRAConfig(quant_type=qt, double_quant=False))
        torch.manual_seed(1)
        w = torch.randn(32, 64) * 0.1
        lin._quantize(w)
        errs[qt] = ((lin.dequantize() - w).norm() / w.norm()).item()
    assert errs[nn.QuantType.INT8] < 0.01 < errs[nn.QuantType.NF4] < errs[nn.QuantType.FP4] < 0.2, errs
    assert nn.PromptInitStrategy.Vocab is nn.PromptInit.Vocab
    pt = nn.PrefixTuning(nn.PrefixTuningConfig(num_prefix_tokens=4, num_layers=2, d_model=32, num_heads=4))
    lp = pt.layer_prefix(1)
    assert isinstance(lp, nn.LayerPrefix) and lp.prefix_key.shape == lp.prefix_value.shape
    cl = nn.CurriculumLearning()
    cl.initialize_samples([0.9, 0.1, 0.5])
    ss = cl.scored_samples(losses=[3.0, 1.0, 2.0])
    assert [s.index for s in ss] == [1, 2, 0] and isinstance(ss[0], nn.ScoredSample) and ss[0].loss == 1.0
    t = nn.ONNXTensor("ids", [2, 2], [1, 2, 3, 4], nn.ONNXDataType.Int64).to_tensor()
    assert t.dtype == torch.int64 and t.shape == (2, 2)
    net = torch.nn.Sequential(torch.nn.Linear(4, 4), torch.nn.BatchNorm1d(4), torch.nn.ReLU())
    opt = nn.InferenceOptimizer()
    opt.optimize(net)
    assert [f.name for f in opt.get_fused_ops()] == ["LinearBN"] and isinstance(opt.get_fused_ops()[0], nn.FusedOp)
    assert AggregatorType.Pool is AggregatorType.Max and GraphSAGELayer is not None
    prof = Profiler(use_cuda_events=False)
    with prof.start("a"):
        pass
    with prof.start("a"):
        pass
    s = prof.get_summary()
    assert isinstance(s, ProfileSummary) and s.total_operations == 2 and s.op_stats["a"].count == 2
    assert len(prof.records) == 2 and isinstance(prof.records[0], ProfileRecord)


def test_graph_layout_hardware_serve_and_model_records():
    from ghost_flow_b200 import models as M
    from ghost_flow_b200 import serve
    from ghost_flow_b200.data import DataLoader, DataLoaderIter, TensorDataset
    from ghost_flow_b200.utils import (ComputeGraph, ElementwiseOp, FusionEngine, FusionOpportunity, HardwareOps,
                                       LayoutOptimizer, MemoryLayout, OperationType, OptimizedLayout, list_devices,
                                       optimize_layout)

    g = ComputeGraph()
    x = g.add_node("Input")
    c = g.add_node("Conv2d", [x])
    b = g.add_node("BatchNorm2d", [c])
    r = g.add_node("ReLU", [b])
    lin = g.add_node("Linear", [r])
    g.add_node("ReLU", [lin])
    g.add_node("Sigmoid", [lin])                       # a second consumer: Linear + ReLU may not fuse
    ops = FusionEngine().find_opportunities(g)
    assert [o.pattern_name for o in ops] == ["ConvBNReLU"] and ops[0].nodes == [c, b, r]
    assert isinstance(ops[0], FusionOpportunity) and ops[0].estimated_speedup > 1 and ops[0].kernel
    lay = optimize_layout((37, 50257), element_size=2, alignment=128, pad_rows=True)
    assert isinstance(lay, OptimizedLayout) and lay.stride == [50304, 1] and lay.aligned_size % 128 == 0
    assert lay.padding == lay.aligned_size - 37 * 50257 * 2
    lo = LayoutOptimizer()
    assert lo.choose_layout(OperationType.Conv2d((3, 3), (1, 1)), (8, 64, 56, 56)) is MemoryLayout.NHWC
    assert OperationType.MatMul(4, 5, 6).params == {"m": 4, "n": 5, "k": 6}
    hw = HardwareOps(list_devices()[0])
    a = torch.tensor([-1.0, 2.0])
    assert torch.equal(hw.elementwise_hw(a, ElementwiseOp.ReLU), torch.tensor([0.0, 2.0]))
    assert torch.equal(hw.elementwise_hw(a, ElementwiseOp.Mul, a), torch.tensor([1.0, 4.0]))
    reg = serve.ModelRegistry("cpu")
    mid = reg.register("double", lambda t: 2 * t, [3], [3])
    info = reg.info(mid)
    assert isinstance(info, serve.ModelInfo) and info.name == "double" and info.input_shape == [3]
    resp = reg.handle(mid, serve.PredictionRequest.from_json({"inputs": [1.0, 2.0, 3.0]}))
    assert isinstance(resp, serve.PredictionResponse) and resp.outputs == [[2.0, 4.0, 6.0]]
    assert resp.to_json()["shape"] == [1, 3]
    cfg = M.CLIPConfig.from_towers(M.CLIPVisionConfig(image_size=32, patch_size=8, hidden_size=64, num_layers=1, num_heads=2),
                                   M.CLIPTextConfig(vocab_size=100, hidden_size=32, num_layers=1, num_heads=2,
                                                    max_position_embeddings=16), embed_dim=24)
    assert cfg.vision_config.hidden_size == 64 and cfg.text_config.max_position_embeddings == 16
    t5 = M.T5Model(M.T5Config.t5_tiny())
    ids = torch.randint(0, 100, (2, 6))
    out = t5(ids, ids[:, :3])
    assert isinstance(out, M.T5Output) and out.last_hidden_state.shape[:2] == (2, 3)
    assert out.encoder_last_hidden_state.shape[:2] == (2, 6)
    it = iter(DataLoader(TensorDataset(torch.arange(10.0)[:, None], torch.arange(10)), batch_size=4))
    assert isinstance(it, DataLoaderIter) and len(it) == 3
    xb, yb = next(it)
    assert xb.shape == (4, 1) and it.current_batch == 1 and len(it) == 2 and len(list(it)) == 2


def test_profiler_exports_a_chrome_trace(tmp_path):
    import json
    import time

    from ghost_flow_b200.utils import Profiler

    prof = Profiler(use_cuda_events=False)
    with prof.start("outer"):
        time.sleep(0.01)
        with prof.start("inner"):
            time.sleep(0.005)
    n = prof.export_chrome_trace(tmp_path / "trace.json")
    ev = json.load(open(tmp_path / "trace.json"))["traceEvents"]
    assert n == 2 and {e["name"] for e in ev} == {"outer", "inner"} and all(e["ph"] == "X" for e in ev)
    outer, inner = (next(e for e in ev if e["name"] == k) for k in ("outer", "inner"))
    assert outer["ts"] <= inner["ts"] and inner["ts"] + inner["dur"] <= outer["ts"] + outer["dur"] + 1e3
    assert outer["dur"] >= 14e3


def test_jit_facade_compiles_unary_chains_and_caches_them():
    from ghost_flow_b200.utils import (CompiledKernel, ComputeGraph, GraphSignature, JitCompiler, OptimizationLevel)

    g = ComputeGraph()
    x = g.add_node("Input")
    a = g.add_node("ReLU", [x])
    b = g.add_node("Tanh", [a])
    g.add_node("Sigmoid", [b])
    jit = JitCompiler()
    k = jit.compile(g, shapes=[(4, 8)])
    assert isinstance(k, CompiledKernel) and k.names == ("relu", "tanh", "sigmoid") and k.fused
    assert isinstance(k.signature, GraphSignature) and k.signature.shapes == ((4, 8),)
    t = torch.randn(4, 8)
    assert torch.allclose(k(t), torch.sigmoid(torch.tanh(torch.relu(t))), atol=1e-6)
    assert jit.compile(g, shapes=[(4, 8)]) is k and jit.hits == 1 and jit.cache_size() == 1
    assert jit.compile(g, shapes=[(2, 8)]) is not k and jit.cache_size() == 2          # another shape, another entry
    slow = JitCompiler(OptimizationLevel.O0).compile(g)
    assert not slow.fused and torch.allclose(slow(t), k(t))
    bad = ComputeGraph()
    i = bad.add_node("Input")
    bad.add_node("Conv2d", [i])
    try:
        jit.compile(bad)
        raise AssertionError("a convolution is not an element-wise chain")
    except ValueError as e:
        assert "Conv2d" in str(e)


def test_storage_guards_and_shared_t5_table():
    import threading
    import time

    from ghost_flow_b200 import models as M
    from ghost_flow_b200.core import Storage, StorageReadGuard, StorageWriteGuard

    st = Storage.from_slice([1.0, 2.0, 3.0])
    assert st.len() == 3 and not st.is_empty() and Storage(torch.float32, 0).is_empty()
    order = []

    def reader():
        with st.read():
            order.append("reader in")

    with st.write() as w:
        assert isinstance(st.write(), StorageWriteGuard) and isinstance(st.read(), StorageReadGuard)
        t = threading.Thread(target=reader)
        t.start()
        time.sleep(0.05)                                    # the reader is blocked on the write guard by now
        w[0] = 10.0
        order.append("writer done")
    t.join(timeout=5)
    assert order == ["writer done", "reader in"]            # the reader waited for the writer
    with st.read() as a, st.read() as b:                    # readers share
        assert float(a[0]) == 10.0 and a.data_ptr() == b.data_ptr()
    t5 = M.T5Model(M.T5Config.t5_tiny())
    assert isinstance(t5.shared, M.T5Embeddings)
    try:
        t5.shared(torch.zeros(3, dtype=torch.long))
        raise AssertionError("1-D ids must be refused")
    except ValueError:
        pass
    c = M.CLIP(M.CLIPConfig.tiny())
    assert isinstance(c.text.layers[0], M.CLIPTextLayer) if hasattr(c, "text") else True


def test_ml_option_enums_are_accepted_where_strings_are():
    import numpy as np

    from ghost_flow_b200 import ml

    X = np.random.RandomState(0).randn(200, 3)
    a = ml.KBinsDiscretizer(4).strategy(ml.BinStrategy.Quantile).encode(ml.BinEncode.Ordinal).fit(X)
    b = ml.KBinsDiscretizer(4).strategy("quantile").fit(X)
    assert np.allclose(a.bin_edges_[0], b.bin_edges_[0]) and a._strategy == "quantile"
    n1 = ml.Normalizer(ml.Norm.L1).fit(X).transform(X)
    assert np.allclose(np.abs(np.asarray(n1.data)).sum(1), 1.0, atol=1e-5)
    assert ml.options.option_value(ml.Scoring.F1) == "f1" and str(ml.SeasonalType.Additive) == "additive"
    assert ml.OPTICSMetric is ml.TSNEMetric


def test_graphed_step_runs_eagerly_without_a_gpu():
    from ghost_flow_b200.utils import GraphedStep

    net = torch.nn.Linear(4, 1)
    opt = torch.optim.SGD(net.parameters(), lr=0.1)

    def train(x, y):
        opt.zero_grad()
        loss = torch.nn.functional.mse_loss(net(x), y)
        loss.backward()
        opt.step()
        return loss.detach()

    x, y = torch.randn(16, 4), torch.randn(16, 1)
    gs = GraphedStep(train, (x, y), warmup=2)
    assert gs.graph is None and len(gs.warmup_outputs) == 2
    losses = [float(gs(x, y)) for _ in range(5)]
    assert gs.replays == 5 and losses[-1] < float(gs.warmup_outputs[0])
    gs.release()
