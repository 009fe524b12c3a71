"""Core value types, the autograd tape / dynamic graph, and the inventory of reference names."""
import importlib
import pkgutil

import pytest
import torch

import ghost_flow_b200 as gf
from ghost_flow_b200.autograd import DynamicContext, DynamicTensor, GradTapeContext, grad_fns, is_recording, record_op


def test_shape_strides_broadcast_offsets():
    s = gf.Shape((2, 1, 4))
    assert s.broadcast_with(gf.Shape((3, 1))) == (2, 3, 4)
    assert s.default_strides() == (4, 4, 1) and s.numel() == 8
    assert s.is_contiguous((4, 4, 1)) and not gf.Shape((2, 3)).is_contiguous((1, 2))
    assert s.offset((1, 0, 2)) == 6
    with pytest.raises(gf.GhostError) as e:
        gf.Shape((2, 3)).broadcast_with(gf.Shape((4, 3)))
    assert e.value.kind is gf.GhostError.Kind.BroadcastError
    assert gf.Cuda(1).torch_device() == torch.device("cuda", 1) and gf.Cpu() == gf.Cpu()
    buf, views = gf.MemoryLayoutOptimizer(64).pack([torch.ones(3), torch.arange(5.0)])
    assert buf.numel() == 128 and views[1].data_ptr() % 64 == buf.data_ptr() % 64 and torch.equal(views[1], torch.arange(5.0))


def test_serializable_round_trip(tmp_path):
    class Box(gf.Serializable):
        def __init__(self):
            self.w = torch.randn(3, 4)

        def state_dict(self):
            return {"w": self.w}

        def load_state_dict(self, s):
            self.w = s["w"]

    a, b = Box(), Box()
    a.save(tmp_path / "box.gf")
    b.load(tmp_path / "box.gf")
    assert torch.equal(a.w, b.w)


def test_tape_and_dynamic_graph_gradients_match_torch():
    a = DynamicTensor(torch.randn(3, 4))
    b = DynamicTensor(torch.randn(4, 2), a.graph)
    y = a.matmul(b).relu().sum()
    y.backward()
    at, bt = a.data.clone().requires_grad_(True), b.data.clone().requires_grad_(True)
    torch.relu(at @ bt).sum().backward()
    assert torch.allclose(a.grad.data, at.grad) and torch.allclose(b.grad.data, bt.grad)
    with DynamicContext.no_grad():
        c = DynamicTensor(torch.ones(2), a.graph)
        assert c.node not in a.graph.nodes
    assert not is_recording()
    with GradTapeContext() as tape:
        assert is_recording()
        x, w = torch.randn(3), torch.randn(3)
        z = x * w
        record_op("mul", [x, w], z, lambda g: grad_fns.mul_backward(g, x, w))
        s = z.exp()
        record_op("exp", [z], s, lambda g: (grad_fns.exp_backward(g, s),))
        gx, gw = tape.gradient(s, [x, w])
    xt = x.clone().requires_grad_(True)
    (xt * w).exp().sum().backward()
    assert torch.allclose(gx, xt.grad) and len(tape.operations) == 2


def test_reference_class_names_are_present():
    have = set(dir(gf))
    for m in pkgutil.walk_packages(gf.__path__, "ghost_flow_b200."):
        if ".csrc" in m.name or ".lib" in m.name:
            continue
        have |= set(dir(importlib.import_module(m.name)))
    names = """Tensor Shape Strides DType GhostError StateDict Serializable MemoryPool MemoryStats MemoryLayoutOptimizer
    TrackedAllocator Profiler ProfileScope Benchmark FusionEngine FusionPattern LayoutOptimizer MemoryLayout
    HardwareBackend HardwareDevice HardwareOps list_devices SparseTensorCOO SparseTensorCSR SparseTensorCSC Device Cpu Cuda
    CudaDevice DeviceGuard CudaStream CudaEvent CudaTimer GpuMemoryPool GpuTensor CudaTensor CuBlas CudaError LaunchConfig
    GradTape GradTapeContext RecordedOp DynamicGraph DynamicContext DynamicTensor
    Linear Conv1d Conv2d Conv3d TransposeConv2d BatchNorm1d BatchNorm2d LayerNorm GroupNorm InstanceNorm Dropout Embedding
    MultiHeadAttention FlashAttention TransformerEncoder TransformerDecoderLayer PositionalEncoding RotaryEmbedding LSTM GRU
    GradScaler AutocastContext CheckpointConfig LoRAConfig LoRALinear QLoRALinear PromptTuningConfig PrefixTuningConfig
    DistillationConfig CurriculumConfig MoEConfig MixtureOfExperts RingAttention StripedRingAttention ZeRoConfig ZeRoOptimizer
    ZeRoStats ZeRoStage DataParallel DistributedDataParallel GradientAccumulator ModelParallel PipelineParallel
    DistributedBackend DistributedConfig FederatedClient FederatedServer SecureAggregation DifferentialPrivacy DPConfig
    DPSGDOptimizer PrivacyAccountant AttackConfig AdversarialTrainingConfig InferenceSession BatchInference ONNXModel
    SGD Adam AdamW StepLR CosineAnnealingLR Dataset DataLoader""".split()
    missing = [n for n in names if n not in have]
    assert not missing, missing


def test_every_kernel_entry_point_named_in_python_is_exported():
    """The ctypes layer looks symbols up lazily, so a missing export would only show on the GPU box: check here that
    every ``lib.gf_*`` attribute the package, the benchmarks and the tests touch exists in the built library."""
    import ctypes
    import glob
    import os
    import re

    from ghost_flow_b200.ops import _lib

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    lib = ctypes.CDLL(str(_lib.lib_path()))
    host = ctypes.CDLL(str(_lib.host_lib_path()))        # host-only entry points (formats, CPU oracle, allocator)
    files = (glob.glob(os.path.join(root, "ghost_flow_b200", "**", "*.py"), recursive=True)
             + glob.glob(os.path.join(root, "benchmarks", "*.py")) + glob.glob(os.path.join(root, "tests", "*.py"))
             + [os.path.join(root, "bench.py"), os.path.join(root, "__graft_entry__.py")])
    names = set()
    for f in files:
        src = open(f).read()
        names |= set(re.findall(r"\.(gf_[a-z0-9_]+)\b", src))
        names |= set(re.findall(r"\"(gf_[a-z0-9_]+)\": \[", src))      # the signature table of ops/_lib.py
    names -= {"gf_cuda", "gf_host"}
    missing = sorted(n for n in names if not hasattr(lib, n) and not hasattr(host, n))
    assert len(names) > 40 and not missing, missing


def test_alias_package_serves_every_submodule():
    import importlib

    import ghost_flow
    import ghost_flow_b200

    for sub in ("nn", "optim", "models", "ml", "ml.tree", "data", "io", "utils", "parallel", "cuda", "serve", "autograd"):
        assert importlib.import_module(f"ghost_flow.{sub}") is importlib.import_module(f"ghost_flow_b200.{sub}")
    from ghost_flow.ml import RandomForestClassifier  # noqa: F401
    from ghost_flow.models import resnet18  # noqa: F401

    assert ghost_flow.Tensor is ghost_flow_b200.Tensor
    with pytest.raises(ModuleNotFoundError):
        importlib.import_module("ghost_flow.no_such_module")


def test_api_advertised_by_the_reference_readme_works():
    """The snippets of the reference's README / PERFORMANCE.md (README.md:217-283, ghost-flow-py/PERFORMANCE.md:24,85),
    which its own bindings do not support, run here."""
    import numpy as np

    import ghost_flow as gf

    model = gf.nn.Sequential([gf.nn.Linear(10, 32), gf.nn.ReLU(), gf.nn.Linear(32, 1)])
    x, y = gf.Tensor.randn(16, 10), gf.Tensor.zeros(16, 1)
    opt = gf.optim.Adam(model.parameters(), lr=1e-2)
    losses = []
    for _ in range(5):
        opt.zero_grad()
        loss = gf.nn.mse_loss(model(x), y)
        loss.backward()
        opt.step()
        losses.append(loss.item())
    assert losses[-1] < losses[0]
    assert ((y - model(x)) ** 2).mean().item() >= 0.0
    assert min((x + 1000).tolist()) > 900
    X = np.random.default_rng(0).normal(size=(80, 4))
    Y = (X[:, 0] > 0).astype(int)
    rf = gf.ml.RandomForest(n_estimators=10, max_depth=4)
    rf.fit(X, Y)
    assert rf.score(X, Y) > 0.9 and len(rf.predict(X).tolist()) == 80
    for name in ("LoRAConfig", "LoRALinear", "FlashAttention", "CurriculumLearning"):
        assert hasattr(gf.nn, name)
    assert hasattr(gf.cuda.Tensor, "randn")
