"""Inference helpers and the legacy model container.

``InferenceConfig``, ``InferenceOptimizer`` (folds BatchNorm into the preceding conv / linear and records the
fusions it applied), ``BatchInference`` (request batching: ``add / is_ready / get_batch / flush``),
``InferenceSession.run / run_batch`` (really executes the module; the reference returns NotImplemented,
ghostflow-nn/src/inference.rs:205-215) and ``warmup_model`` (inference.rs:239-264).

``ONNXModel / ONNXGraph / ONNXNode / ONNXTensor`` with ``save / load`` in the reference's private container
(magic ``b"ONNX"``, not protobuf: ghostflow-nn/src/onnx.rs:86-130) for reading its files; real ONNX export goes
through ``torch.onnx``.
"""
from __future__ import annotations

import enum
import struct
import time
from dataclasses import dataclass, field

import torch

from .module import Module


@dataclass
class InferenceConfig:
    batch_size: int = 32
    max_wait_ms: float = 5.0
    fuse_operators: bool = True
    fold_constants: bool = True
    use_half_precision: bool = False
    num_threads: int = 1
    use_cuda_graph: bool = False     # replay CUDA inputs from a captured graph (see CudaGraphRunner)


@dataclass
class FusedOp:
    """A fusion the optimizer performed: its name and the operators it replaced
    (ghostflow-nn/src/inference.rs:45-50; there the list is a fixed announcement, here it records what was done)."""
    name: str
    ops: list


class InferenceOptimizer:
    def __init__(self, config: InferenceConfig | None = None):
        self.config = config or InferenceConfig()
        self.applied: list[str] = []
        self.fused_ops: list = []

    def get_fused_ops(self) -> list:
        return list(self.fused_ops)

    @torch.no_grad()
    def optimize(self, model: torch.nn.Module) -> torch.nn.Module:
        """Returns the model in eval mode with Conv/Linear + BatchNorm pairs folded (in ``Sequential``-like
        containers) and, if requested, cast to bf16."""
        model.eval()
        if self.config.fuse_operators:
            self._fold_bn(model)
        if self.config.use_half_precision:
            model.to(torch.bfloat16)
            self.applied.append("cast_bf16")
        return model

    def _fold_bn(self, module):
        from .conv import Conv2d
        from .layers import BatchNorm1d, BatchNorm2d, Linear

        children = list(module.named_children())
        for (n1, a), (n2, b) in zip(children, children[1:]):
            if isinstance(a, (Conv2d, torch.nn.Conv2d, Linear, torch.nn.Linear)) and isinstance(
                    b, (BatchNorm1d, BatchNorm2d, torch.nn.BatchNorm1d, torch.nn.BatchNorm2d)):
                scale = b.weight / torch.sqrt(b.running_var + b.eps) if b.weight is not None else \
                    1.0 / torch.sqrt(b.running_var + b.eps)
                a.weight.mul_(scale.view(-1, *[1] * (a.weight.dim() - 1)))
                bias = a.bias if a.bias is not None else torch.zeros_like(b.running_mean)
                new_bias = (bias - b.running_mean) * scale + (b.bias if b.bias is not None else 0)
                a.bias = torch.nn.Parameter(new_bias)
                self._replace(module, n2, torch.nn.Identity())
                self.applied.append(f"fold_bn:{n1}+{n2}")
                self.fused_ops.append(FusedOp("ConvBN" if a.weight.dim() == 4 else "LinearBN",
                                              [type(a).__name__, type(b).__name__]))
        for _, child in module.named_children():
            self._fold_bn(child)

    @staticmethod
    def _replace(module, name, new):
        if isinstance(module, (torch.nn.Sequential, torch.nn.ModuleList)) and name.isdigit():
            module[int(name)] = new
        else:
            setattr(module, name, new)

    def get_fusions(self):
        return list(self.applied)


def _map_tensors(obj, fn):
    """Applies ``fn`` to every torch tensor inside tuples / lists / dicts / dataclasses / named tuples."""
    import dataclasses

    from ..tensor import Tensor

    if isinstance(obj, torch.Tensor):
        return fn(obj)
    if isinstance(obj, Tensor):
        return Tensor(fn(obj.data))
    if isinstance(obj, tuple) and hasattr(obj, "_fields"):
        return type(obj)(*[_map_tensors(o, fn) for o in obj])
    if isinstance(obj, (tuple, list)):
        return type(obj)(_map_tensors(o, fn) for o in obj)
    if isinstance(obj, dict):
        return {k: _map_tensors(v, fn) for k, v in obj.items()}
    if dataclasses.is_dataclass(obj) and not isinstance(obj, type):
        return dataclasses.replace(obj, **{f.name: _map_tensors(getattr(obj, f.name), fn)
                                           for f in dataclasses.fields(obj)})
    return obj


class CudaGraphRunner:
    """Replays a forward pass from a CUDA graph, so that a launch-bound model costs one launch per call.

    ``runner = CudaGraphRunner(fn)``; ``runner(x, ...)`` takes CUDA tensors. The first call with a new combination
    of input shapes and dtypes runs ``fn`` a few times eagerly on a side stream (so that every lazily created
    workspace exists), then captures it with the inputs held in static buffers; later calls copy their inputs into
    those buffers and replay. ``fn`` must be free of autograd, host synchronisation and data-dependent control
    flow, and its parameters must stay where they are (rebuild the runner after ``model.to(...)``). Results are
    cloned out of the graph's static outputs unless ``clone_outputs=False`` (then they are overwritten by the
    next call). The library's own kernels launch on the current stream and keep their tensor maps in kernel
    arguments, so they are captured like any other launch.
    """

    def __init__(self, fn, warmup: int = 3, clone_outputs: bool = True, max_graphs: int = 16):
        self.fn, self.warmup, self.clone_outputs, self.max_graphs = fn, warmup, clone_outputs, max_graphs
        self._cache: dict = {}

    def _capture(self, inputs):
        static_in = [t.clone() for t in inputs]
        side = torch.cuda.Stream(device=inputs[0].device)
        side.wait_stream(torch.cuda.current_stream(inputs[0].device))
        with torch.cuda.stream(side), torch.no_grad():
            for _ in range(max(self.warmup, 1)):
                self.fn(*static_in)
        torch.cuda.current_stream(inputs[0].device).wait_stream(side)
        torch.cuda.synchronize(inputs[0].device)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph), torch.no_grad():
            static_out = self.fn(*static_in)
        return static_in, graph, static_out

    def __call__(self, *inputs):
        from ..tensor import Tensor

        inputs = [t.data if isinstance(t, Tensor) else t for t in inputs]
        key = tuple((tuple(t.shape), t.dtype, t.device.index) for t in inputs)
        entry = self._cache.get(key)
        if entry is None:
            if len(self._cache) >= self.max_graphs:
                self._cache.pop(next(iter(self._cache)))
            entry = self._cache[key] = self._capture(inputs)
        static_in, graph, static_out = entry
        for s, t in zip(static_in, inputs):
            s.copy_(t)
        graph.replay()
        return _map_tensors(static_out, torch.clone) if self.clone_outputs else static_out


class BatchInference:
    """Collects single requests into batches of ``batch_size`` (or whatever is there after ``max_wait_ms``)."""

    def __init__(self, batch_size: int = 32, max_wait_ms: float = 5.0):
        self.batch_size, self.max_wait_ms = batch_size, max_wait_ms
        self.pending: list = []
        self.first_at: float | None = None

    def add(self, x):
        if not self.pending:
            self.first_at = time.monotonic()
        self.pending.append(x)

    def is_ready(self) -> bool:
        if len(self.pending) >= self.batch_size:
            return True
        return bool(self.pending) and (time.monotonic() - self.first_at) * 1e3 >= self.max_wait_ms

    def get_batch(self):
        n = min(self.batch_size, len(self.pending))
        items, self.pending = self.pending[:n], self.pending[n:]
        self.first_at = time.monotonic() if self.pending else None
        return torch.stack(items) if items else None

    def flush(self):
        out = []
        while self.pending:
            out.append(self.get_batch())
        return out


class InferenceSession:
    def __init__(self, model: torch.nn.Module, config: InferenceConfig | None = None):
        self.config = config or InferenceConfig()
        self.optimizer = InferenceOptimizer(self.config)
        self.model = self.optimizer.optimize(model)
        self._graphs = CudaGraphRunner(self.model) if self.config.use_cuda_graph else None

    @torch.no_grad()
    def run(self, x):
        from ..tensor import Tensor

        data = x.data if isinstance(x, Tensor) else x
        if self._graphs is not None and torch.is_tensor(data) and data.is_cuda:
            out = self._graphs(data)
            return Tensor(out) if isinstance(x, Tensor) and torch.is_tensor(out) else out
        if isinstance(x, Tensor):
            return Tensor(self.model(x.data))
        return self.model(x)

    def run_batch(self, inputs):
        batcher = BatchInference(self.config.batch_size, 0.0)
        for x in inputs:
            batcher.add(x)
        outs = []
        for b in batcher.flush():
            outs.extend(self.run(b).unbind(0))
        return outs


def warmup_model(fn, input_shape, iterations: int = 10, device=None) -> float:
    """Average milliseconds per call of ``fn`` on a random input of ``input_shape`` (CUDA events on a GPU)."""
    x = torch.randn(*input_shape, device=device)
    fn(x)
    if x.is_cuda:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(iterations):
            fn(x)
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / iterations
    t0 = time.perf_counter()
    for _ in range(iterations):
        fn(x)
    return (time.perf_counter() - t0) * 1e3 / iterations


# ------------------------------------------------------------------------------------------- legacy "ONNX" container
class ONNXDataType(enum.Enum):
    """Element types of the container (ghostflow-nn/src/onnx.rs:11-19)."""
    Float32 = "float32"
    Float64 = "float64"
    Int32 = "int32"
    Int64 = "int64"
    Uint8 = "uint8"

    def torch_dtype(self):
        return getattr(torch, self.value)


@dataclass
class ONNXTensor:
    name: str
    dims: list
    data: list
    dtype: "ONNXDataType" = None

    def __post_init__(self):
        if self.dtype is None:
            self.dtype = ONNXDataType.Float32

    def to_tensor(self):
        return torch.tensor(self.data, dtype=self.dtype.torch_dtype()).reshape(self.dims)


@dataclass
class ONNXAttribute:
    name: str
    value: str


@dataclass
class ONNXNode:
    name: str
    op_type: str
    inputs: list = field(default_factory=list)
    outputs: list = field(default_factory=list)
    attributes: list = field(default_factory=list)


@dataclass
class ONNXGraph:
    name: str = "graph"
    nodes: list = field(default_factory=list)
    inputs: list = field(default_factory=list)
    outputs: list = field(default_factory=list)
    initializers: list = field(default_factory=list)


def tensor_to_onnx(name: str, t: torch.Tensor) -> ONNXTensor:
    t = getattr(t, "data", t) if not isinstance(t, torch.Tensor) else t
    return ONNXTensor(name, list(t.shape), t.detach().float().reshape(-1).tolist())


def onnx_to_tensor(t: ONNXTensor) -> torch.Tensor:
    return t.to_tensor()


def _ws(b: bytearray, s: str):
    e = s.encode()
    b += struct.pack("<I", len(e)) + e


def _rs(buf, off):
    (n,) = struct.unpack_from("<I", buf, off)
    return buf[off + 4:off + 4 + n].decode(), off + 4 + n


@dataclass
class ONNXModel:
    """Graph + weights in the private ``b"ONNX"`` container: magic, u32 ir_version, producer string, graph name,
    then counted lists of nodes, inputs, outputs and initialisers (strings are u32 length + bytes)."""
    ir_version: int = 8
    producer_name: str = "ghostflow"
    graph: ONNXGraph = field(default_factory=ONNXGraph)

    def save(self, path):
        b = bytearray(b"ONNX")
        b += struct.pack("<I", self.ir_version)
        _ws(b, self.producer_name)
        g = self.graph
        _ws(b, g.name)
        b += struct.pack("<I", len(g.nodes))
        for n in g.nodes:
            _ws(b, n.name)
            _ws(b, n.op_type)
            for lst in (n.inputs, n.outputs):
                b += struct.pack("<I", len(lst))
                for s in lst:
                    _ws(b, s)
            b += struct.pack("<I", len(n.attributes))
            for a in n.attributes:
                _ws(b, a.name)
                _ws(b, str(a.value))
        for lst in (g.inputs, g.outputs):
            b += struct.pack("<I", len(lst))
            for s in lst:
                _ws(b, s)
        b += struct.pack("<I", len(g.initializers))
        for t in g.initializers:
            _ws(b, t.name)
            b += struct.pack("<I", len(t.dims)) + struct.pack(f"<{len(t.dims)}Q", *t.dims)
            b += struct.pack("<Q", len(t.data)) + struct.pack(f"<{len(t.data)}f", *t.data)
        with open(path, "wb") as f:
            f.write(b)

    @classmethod
    def load(cls, path):
        buf = open(path, "rb").read()
        if buf[:4] != b"ONNX":
            raise IOError("not a GhostFlow ONNX container")
        (ir,) = struct.unpack_from("<I", buf, 4)
        off = 8
        prod, off = _rs(buf, off)
        gname, off = _rs(buf, off)
        g = ONNXGraph(gname)
        (nn,) = struct.unpack_from("<I", buf, off); off += 4
        for _ in range(nn):
            name, off = _rs(buf, off)
            op, off = _rs(buf, off)
            lists = []
            for _k in range(2):
                (c,) = struct.unpack_from("<I", buf, off); off += 4
                cur = []
                for _j in range(c):
                    s, off = _rs(buf, off)
                    cur.append(s)
                lists.append(cur)
            (na,) = struct.unpack_from("<I", buf, off); off += 4
            attrs = []
            for _j in range(na):
                an, off = _rs(buf, off)
                av, off = _rs(buf, off)
                attrs.append(ONNXAttribute(an, av))
            g.nodes.append(ONNXNode(name, op, lists[0], lists[1], attrs))
        for target in (g.inputs, g.outputs):
            (c,) = struct.unpack_from("<I", buf, off); off += 4
            for _j in range(c):
                s, off = _rs(buf, off)
                target.append(s)
        (ni,) = struct.unpack_from("<I", buf, off); off += 4
        for _ in range(ni):
            name, off = _rs(buf, off)
            (nd,) = struct.unpack_from("<I", buf, off); off += 4
            dims = list(struct.unpack_from(f"<{nd}Q", buf, off)); off += 8 * nd
            (ln,) = struct.unpack_from("<Q", buf, off); off += 8
            data = list(struct.unpack_from(f"<{ln}f", buf, off)); off += 4 * ln
            g.initializers.append(ONNXTensor(name, dims, data))
        return cls(ir, prod, g)

    @classmethod
    def from_sequential(cls, model: torch.nn.Module, input_name="input"):
        """Describes a Linear/activation stack as Gemm / Relu / ... nodes with its weights as initialisers."""
        g = ONNXGraph("main", inputs=[input_name])
        cur = input_name
        for i, (name, m) in enumerate(model.named_modules()):
            if name == "" or list(m.children()):
                continue
            out = f"t{i}"
            if hasattr(m, "weight") and getattr(m, "weight", None) is not None and m.weight.dim() == 2:
                g.initializers.append(tensor_to_onnx(f"{name}.weight", m.weight))
                ins = [cur, f"{name}.weight"]
                if getattr(m, "bias", None) is not None:
                    g.initializers.append(tensor_to_onnx(f"{name}.bias", m.bias))
                    ins.append(f"{name}.bias")
                g.nodes.append(ONNXNode(name, "Gemm", ins, [out], [ONNXAttribute("transB", "1")]))
            else:
                g.nodes.append(ONNXNode(name, type(m).__name__, [cur], [out]))
            cur = out
        g.outputs = [cur]
        return cls(graph=g)
