"""Runtime utilities with the reference's names.

* ``Profiler / ProfileScope / Benchmark / global_profiler / profile`` (ghostflow-core/src/profiler.rs:10-305): same
  API, but GPU work is timed with CUDA events on the current stream (plus NVTX ranges) and the profiler can hook
  every ``Module.__call__`` (the reference's profiler is hooked into nothing).
* ``MemoryPool / MemoryStats / TrackedAllocator`` (ghostflow-core/src/memory.rs:9-239): pinned host staging pool with
  size buckets and the same counters.
* ``FusionEngine`` (ghostflow-core/src/fusion.rs:108-229): same pattern names; here ``fuse`` returns which kernel of
  this library implements each matched pattern.
* ``MemoryLayout / LayoutOptimizer / DeviceInfo`` (ghostflow-core/src/layout/mod.rs:10-226).
* ``HardwareBackend / HardwareDevice / list_devices / HardwareOps`` (ghostflow-core/src/hardware.rs:15-414): the enum
  keeps every label for API parity; only CPU and CUDA devices are ever reported.
* ``SparseTensorCOO / CSR / CSC`` (ghostflow-core/src/sparse.rs:14-424) over torch sparse tensors.
* ``StepLogger``: JSONL training metrics.
"""
from __future__ import annotations

import contextlib
import enum
import json
import math
import os
import statistics
import time
from dataclasses import dataclass, field

import torch

from .graphs import GraphedStep  # noqa: F401


# =========================================================================== profiler
@dataclass
class OpStats:
    count: int = 0
    total_ms: float = 0.0
    min_ms: float = math.inf
    max_ms: float = 0.0

    @property
    def avg_ms(self):
        return self.total_ms / self.count if self.count else 0.0


class ProfileScope:
    def __init__(self, profiler, name: str):
        self.profiler, self.name = profiler, name

    def __enter__(self):
        self.cuda = torch.cuda.is_available() and self.profiler.use_cuda_events
        if self.cuda:
            torch.cuda.nvtx.range_push(self.name)
            self.e0, self.e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            self.e0.record()
        self.t0 = time.perf_counter()
        return self

    def __exit__(self, *a):
        if self.cuda:
            self.e1.record()
            torch.cuda.nvtx.range_pop()
            self.profiler._pending.append((self.name, self.e0, self.e1, self.t0))
        else:
            self.profiler._record(self.name, (time.perf_counter() - self.t0) * 1e3, self.t0)
        return False


@dataclass
class ProfileRecord:
    """One timed scope (ghostflow-core/src/profiler.rs:141-146)."""
    name: str
    duration_ms: float
    start_ms: float = 0.0        # host time of the scope's entry, relative to the profiler's creation


@dataclass
class ProfileSummary:
    """Totals per operation name (ghostflow-core/src/profiler.rs:170-175)."""
    total_operations: int
    op_stats: dict


class Profiler:
    def __init__(self, use_cuda_events: bool = True, keep_records: int = 100_000):
        self.enabled = True
        self.use_cuda_events = use_cuda_events
        self.stats: dict[str, OpStats] = {}
        self._pending = []
        self.records: list = []            # the last ``keep_records`` scopes in completion order
        self._keep = keep_records
        self._t_origin = time.perf_counter()

    def start(self, name: str) -> ProfileScope:
        return ProfileScope(self, name)

    scope = start

    def _record(self, name, ms, t0=None):
        if len(self.records) < self._keep:
            self.records.append(ProfileRecord(name, ms, 0.0 if t0 is None else (t0 - self._t_origin) * 1e3))
        s = self.stats.setdefault(name, OpStats())
        s.count += 1
        s.total_ms += ms
        s.min_ms, s.max_ms = min(s.min_ms, ms), max(s.max_ms, ms)

    def _flush(self):
        if self._pending:
            torch.cuda.synchronize()
            for name, e0, e1, t0 in self._pending:
                self._record(name, e0.elapsed_time(e1), t0)
            self._pending = []

    def summary(self) -> dict:
        self._flush()
        return {k: {"count": v.count, "total_ms": v.total_ms, "avg_ms": v.avg_ms, "min_ms": v.min_ms, "max_ms": v.max_ms}
                for k, v in self.stats.items()}

    def get_summary(self) -> ProfileSummary:
        self._flush()
        return ProfileSummary(sum(v.count for v in self.stats.values()), dict(self.stats))

    def export_chrome_trace(self, path) -> int:
        """Writes the recorded scopes as a Chrome / Perfetto trace (``chrome://tracing``, ui.perfetto.dev): one
        complete event per scope, placed at the host time of its entry with its measured duration (device time for
        CUDA-event scopes). Returns the number of events."""
        self._flush()
        events = [{"name": r.name, "ph": "X", "ts": r.start_ms * 1e3, "dur": r.duration_ms * 1e3, "pid": os.getpid(),
                   "tid": 0, "cat": "ghost_flow"} for r in self.records]
        with open(path, "w") as f:
            json.dump({"traceEvents": events, "displayTimeUnit": "ms"}, f)
        return len(events)

    def print_summary(self):
        rows = sorted(self.summary().items(), key=lambda kv: -kv[1]["total_ms"])
        print(f"{'op':<32}{'count':>8}{'total ms':>12}{'avg ms':>10}{'min ms':>10}{'max ms':>10}")
        for k, v in rows:
            print(f"{k:<32}{v['count']:>8}{v['total_ms']:>12.3f}{v['avg_ms']:>10.3f}{v['min_ms']:>10.3f}{v['max_ms']:>10.3f}")

    def reset(self):
        self.stats, self._pending, self.records = {}, [], []

    def hook_modules(self, enable: bool = True):
        """Times every ``ghost_flow_b200.nn.Module`` call under its class name."""
        from ..nn.module import Module

        Module._profile_hook = self.start if enable else None


_GLOBAL = None


def global_profiler() -> Profiler:
    global _GLOBAL
    if _GLOBAL is None:
        _GLOBAL = Profiler()
    return _GLOBAL


@contextlib.contextmanager
def profile(name: str):
    with global_profiler().start(name):
        yield


@dataclass
class BenchmarkResult:
    name: str
    mean: float
    median: float
    min: float
    max: float
    std_dev: float
    iterations: int

    def __str__(self):
        return (f"{self.name}: mean {self.mean:.4f} ms, median {self.median:.4f}, min {self.min:.4f}, "
                f"max {self.max:.4f}, std {self.std_dev:.4f} ({self.iterations} iters)")


class Benchmark:
    """``Benchmark(name).warmup(n).iterations(m).run(fn)``; CUDA events when a GPU is present."""

    def __init__(self, name: str):
        self.name, self._warmup, self._iters = name, 3, 10

    def warmup(self, n: int):
        self._warmup = n
        return self

    def iterations(self, n: int):
        self._iters = n
        return self

    def run(self, fn) -> BenchmarkResult:
        for _ in range(self._warmup):
            fn()
        times = []
        cuda = torch.cuda.is_available()
        for _ in range(self._iters):
            if cuda:
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                torch.cuda.synchronize()
                e0.record()
                fn()
                e1.record()
                torch.cuda.synchronize()
                times.append(e0.elapsed_time(e1))
            else:
                t0 = time.perf_counter()
                fn()
                times.append((time.perf_counter() - t0) * 1e3)
        return BenchmarkResult(self.name, statistics.fmean(times), statistics.median(times), min(times), max(times),
                               statistics.pstdev(times) if len(times) > 1 else 0.0, self._iters)


# =========================================================================== host memory pool
@dataclass
class MemoryStats:
    total_allocations: int = 0
    reused_allocations: int = 0
    current_usage: int = 0
    peak_usage: int = 0

    def reuse_rate(self) -> float:
        return self.reused_allocations / self.total_allocations if self.total_allocations else 0.0


@dataclass
class AllocationStats:
    """Counters of a tracked allocator (ghostflow-core/src/memory.rs:214-239)."""
    allocations: int = 0
    deallocations: int = 0
    total_allocated: int = 0
    current_allocated: int = 0
    peak_allocated: int = 0

    def current_mb(self) -> float:
        return self.current_allocated / (1024.0 * 1024.0)

    def peak_mb(self) -> float:
        return self.peak_allocated / (1024.0 * 1024.0)

    def total_mb(self) -> float:
        return self.total_allocated / (1024.0 * 1024.0)


class MemoryPool:
    """Size-bucketed (power of two) reuse of pinned host staging buffers."""

    def __init__(self, pinned: bool = False):
        self.pinned = pinned and torch.cuda.is_available()
        self.free: dict[int, list] = {}
        self.stats = MemoryStats()

    @staticmethod
    def _bucket(nbytes: int) -> int:
        return 1 << max(6, (max(1, nbytes) - 1).bit_length())

    def allocate(self, nbytes: int) -> torch.Tensor:
        b = self._bucket(nbytes)
        self.stats.total_allocations += 1
        lst = self.free.get(b)
        if lst:
            self.stats.reused_allocations += 1
            buf = lst.pop()
        else:
            buf = torch.empty(b, dtype=torch.uint8, pin_memory=self.pinned)
        self.stats.current_usage += b
        self.stats.peak_usage = max(self.stats.peak_usage, self.stats.current_usage)
        return buf

    def deallocate(self, buf: torch.Tensor):
        b = buf.numel()
        self.free.setdefault(b, []).append(buf)
        self.stats.current_usage -= b

    def clear(self):
        self.free.clear()

    def get_stats(self) -> MemoryStats:
        return self.stats


class TrackedAllocator:
    """Counts allocations made through it (for tests and leak hunting)."""

    def __init__(self):
        self.allocations, self.deallocations, self.bytes_allocated = 0, 0, 0
        self._current = self._peak = 0

    def allocate(self, shape, dtype=torch.float32, device="cpu"):
        t = torch.empty(shape, dtype=dtype, device=device)
        self.allocations += 1
        n = t.numel() * t.element_size()
        self.bytes_allocated += n
        self._current += n
        self._peak = max(self._peak, self._current)
        return t

    def free(self, t):
        self.deallocations += 1
        self._current -= t.numel() * t.element_size()

    def allocation_stats(self) -> AllocationStats:
        return AllocationStats(self.allocations, self.deallocations, self.bytes_allocated, self._current, self._peak)

    def stats(self):
        return {"allocations": self.allocations, "deallocations": self.deallocations,
                "bytes_allocated": self.bytes_allocated}


# =========================================================================== fusion patterns
class FusionPattern(enum.Enum):
    ConvBNReLU = "ConvBNReLU"
    LinearReLU = "LinearReLU"
    GEMM = "GEMM"
    AddReLU = "AddReLU"
    FMA = "FMA"
    BNReLU = "BNReLU"
    LinearResidual = "LinearResidual"
    NormResidual = "NormResidual"
    GateUpSwiGLU = "GateUpSwiGLU"
    SoftmaxXent = "SoftmaxXent"


_PATTERNS = [
    (("Conv2d", "BatchNorm2d", "ReLU"), FusionPattern.ConvBNReLU, "gf_conv_bn_relu", 3.0),
    (("Linear", "ReLU"), FusionPattern.LinearReLU, "gf_gemm_bf16 + gf_unary_fwd", 1.3),
    (("MatMul", "Add"), FusionPattern.GEMM, "gf_gemm_bf16 (bias epilogue)", 1.5),
    (("Linear", "Add"), FusionPattern.LinearResidual, "gf_gemm_bf16 (residual epilogue)", 1.4),
    (("Add", "ReLU"), FusionPattern.AddReLU, "gf_op_chain", 1.8),
    (("Mul", "Add"), FusionPattern.FMA, "gf_binary", 1.5),
    (("BatchNorm2d", "ReLU"), FusionPattern.BNReLU, "gf_conv_bn_relu", 1.6),
    (("Add", "RMSNorm"), FusionPattern.NormResidual, "gf_rmsnorm_fwd (residual input)", 1.8),
    (("Linear", "SwiGLU"), FusionPattern.GateUpSwiGLU, "gf_gemm_bf16 + gf_swiglu_fwd", 1.2),
    (("Softmax", "CrossEntropy"), FusionPattern.SoftmaxXent, "gf_xent_fused", 2.0),
]


@dataclass
class GraphNode:
    """One operation of a :class:`ComputeGraph` (ghostflow-core/src/fusion.rs:22-30)."""
    id: int
    op: str
    inputs: list = field(default_factory=list)


@dataclass
class FusionOpportunity:
    """A run of nodes that one kernel of this library can execute (ghostflow-core/src/fusion.rs:243-249)."""
    pattern_name: str
    nodes: list
    estimated_speedup: float
    kernel: str = ""


class ComputeGraph:
    """A small op graph for fusion analysis (ghostflow-core/src/fusion.rs:32-80): nodes are added in topological
    order with the ids of their inputs."""

    def __init__(self):
        self.nodes: list = []

    def add_node(self, op: str, inputs=()) -> int:
        self.nodes.append(GraphNode(len(self.nodes), op, list(inputs)))
        return len(self.nodes) - 1

    def consumers(self, node_id: int) -> list:
        return [n.id for n in self.nodes if node_id in n.inputs]

    def chains(self) -> list:
        """Maximal runs of nodes in which every node is the only consumer of its predecessor (only such runs can be
        fused without keeping an intermediate alive)."""
        out, seen = [], set()
        for n in self.nodes:
            if n.id in seen:
                continue
            run, cur = [n.id], n
            seen.add(n.id)
            while True:
                cons = self.consumers(cur.id)
                if len(cons) != 1 or self.nodes[cons[0]].inputs[0] != cur.id or cons[0] in seen:
                    break
                cur = self.nodes[cons[0]]
                run.append(cur.id)
                seen.add(cur.id)
            out.append(run)
        return out


class FusionEngine:
    def __init__(self):
        self.fused: list = []

    def find_opportunities(self, graph: "ComputeGraph") -> list:
        """:class:`FusionOpportunity` records for every pattern match inside a single-consumer chain of ``graph``."""
        out = []
        for run in graph.chains():
            names = [graph.nodes[i].op for i in run]
            for start, pat in self.analyze(names):
                n = next(len(p[0]) for p in _PATTERNS if p[1] == pat)
                out.append(FusionOpportunity(pat.value, run[start:start + n], self.estimate_speedup(pat),
                                             self.kernel_for(pat)))
        return out

    def analyze(self, ops: list[str]) -> list:
        """Finds fusable runs in a list of op names; returns ``[(start_index, pattern)]`` (longest match first)."""
        out, i = [], 0
        while i < len(ops):
            hit = None
            for names, pat, _, _ in sorted(_PATTERNS, key=lambda p: -len(p[0])):
                if tuple(ops[i:i + len(names)]) == names:
                    hit = (i, pat, len(names))
                    break
            if hit:
                out.append((hit[0], hit[1]))
                i += hit[2]
            else:
                i += 1
        return out

    def estimate_speedup(self, pattern: FusionPattern) -> float:
        return next(p[3] for p in _PATTERNS if p[1] == pattern)

    def kernel_for(self, pattern: FusionPattern) -> str:
        return next(p[2] for p in _PATTERNS if p[1] == pattern)

    def fuse(self, ops: list[str]) -> list:
        self.fused = [{"index": i, "pattern": p.value, "kernel": self.kernel_for(p)} for i, p in self.analyze(ops)]
        return self.fused

    def analyze_module(self, module: torch.nn.Module) -> list:
        return self.fuse([type(m).__name__ for m in module.modules() if not list(m.children())])


# =========================================================================== "JIT": cached fused element-wise chains
class OptimizationLevel(enum.Enum):
    """Kept for the reference's surface (ghostflow-core/src/jit/mod.rs:39-46). There is nothing to tune: a chain is
    one launch of the op-chain kernel at every level; O0 runs the operations one by one."""
    O0 = 0
    O1 = 1
    O2 = 2
    O3 = 3


@dataclass(frozen=True)
class GraphSignature:
    """Cache key of a compiled graph: operation names and input shapes (ghostflow-core/src/jit/mod.rs:26-31)."""
    ops: tuple
    shapes: tuple = ()


class CompiledKernel:
    """What :meth:`JitCompiler.compile` returns: call it with the input tensor."""

    def __init__(self, signature: GraphSignature, names: tuple, fused: bool):
        self.signature, self.names, self.fused = signature, names, fused
        self.calls = 0

    def __call__(self, x):
        from .. import ops

        self.calls += 1
        if self.fused:
            return ops.op_chain(x, list(self.names))          # one pass over memory (gf_op_chain on the GPU)
        for n in self.names:
            x = ops.unary(x, n)
        return x

    execute = __call__


class JitCompiler:
    """The reference generates CUDA source for a chain of element-wise operations and compiles it with nvcc at run
    time (ghostflow-core/src/jit/mod.rs:48-150; the generated kernel is never launched there). Here the same job is
    done without a compiler at run time: the library's op-chain kernel takes up to eight unary operations as launch
    arguments and applies them in one pass, so "compiling" a graph means checking that it is such a chain and
    caching the callable under its signature. Graphs with other operations are refused with the reason."""

    _NAMES = {"relu": "relu", "gelu": "gelu", "sigmoid": "sigmoid", "tanh": "tanh", "silu": "silu", "exp": "exp",
              "neg": "neg", "abs": "abs", "sqrt": "sqrt", "square": "square"}

    def __init__(self, optimization_level: OptimizationLevel = OptimizationLevel.O3):
        self.optimization_level = optimization_level
        self.cache: dict = {}
        self.hits = self.misses = 0

    def compute_signature(self, graph: "ComputeGraph", shapes=()) -> GraphSignature:
        return GraphSignature(tuple(n.op for n in graph.nodes), tuple(tuple(s) for s in shapes))

    def compile(self, graph: "ComputeGraph", shapes=()) -> CompiledKernel:
        from ..ops.fused import OPS

        sig = self.compute_signature(graph, shapes)
        if sig in self.cache:
            self.hits += 1
            return self.cache[sig]
        self.misses += 1
        body = [n for n in graph.nodes if n.op.lower() not in ("input", "output")]
        names = []
        for i, n in enumerate(body):
            key = self._NAMES.get(n.op.lower())
            if key is None or key not in OPS:
                raise ValueError(f"cannot fuse operation {n.op!r}: only chains of unary element-wise operations "
                                 f"({', '.join(sorted(k for k in self._NAMES if k in OPS))}) compile to one kernel")
            if i and n.inputs and n.inputs[0] != body[i - 1].id:
                raise ValueError("the graph is not a single chain")
            names.append(key)
        if not names or len(names) > 8:
            raise ValueError("a chain needs between one and eight operations")
        kern = CompiledKernel(sig, tuple(names), fused=self.optimization_level != OptimizationLevel.O0)
        self.cache[sig] = kern
        return kern

    def clear_cache(self):
        self.cache.clear()

    def cache_size(self) -> int:
        return len(self.cache)


# =========================================================================== layouts
class MemoryLayout(enum.Enum):
    NCHW = "NCHW"
    NHWC = "NHWC"
    CHWN = "CHWN"
    BSF = "BSF"
    SBF = "SBF"


@dataclass
class DeviceInfo:
    name: str = "NVIDIA B200"
    compute_capability: tuple = (10, 0)
    memory_bandwidth_gbs: float = 7700.0
    num_sms: int = 148
    l2_bytes: int = 126 * 1024 * 1024
    has_tensor_cores: bool = True

    @classmethod
    def current(cls):
        if torch.cuda.is_available():
            p = torch.cuda.get_device_properties(0)
            return cls(p.name, (p.major, p.minor), 7700.0 if p.major >= 10 else 2000.0, p.multi_processor_count,
                       getattr(p, "L2_cache_size", 0), p.major >= 7)
        return cls("cpu", (0, 0), 100.0, 1, 0, False)


@dataclass
class OperationType:
    """What a layout is chosen for (ghostflow-core/src/layout/mod.rs:56-66): a kind plus its parameters. Build with
    the class methods, e.g. ``OperationType.Conv2d((3, 3), (1, 1))`` or ``OperationType.MatMul(4096, 4096, 4096)``."""
    kind: str
    params: dict = field(default_factory=dict)

    @classmethod
    def Conv2d(cls, kernel=(3, 3), stride=(1, 1)): return cls("Conv2d", {"kernel": tuple(kernel), "stride": tuple(stride)})
    @classmethod
    def MatMul(cls, m, n, k): return cls("MatMul", {"m": m, "n": n, "k": k})
    @classmethod
    def BatchNorm(cls): return cls("BatchNorm")
    @classmethod
    def LayerNorm(cls): return cls("LayerNorm")
    @classmethod
    def Attention(cls, heads, seq_len): return cls("Attention", {"heads": heads, "seq_len": seq_len})
    @classmethod
    def ElementWise(cls): return cls("ElementWise")
    @classmethod
    def Pooling(cls): return cls("Pooling")


@dataclass
class OptimizedLayout:
    """Padded allocation plan of a tensor (ghostflow-core/src/memory.rs:156-163)."""
    original_size: int
    aligned_size: int
    padding: int
    stride: list


def optimize_layout(shape, element_size: int = 4, alignment: int = 256, pad_rows: bool = False) -> OptimizedLayout:
    """Row-major strides of ``shape`` (in elements) with the total size rounded up to ``alignment`` bytes; with
    ``pad_rows`` the innermost row is padded to the alignment too (what TMA tensor maps and 16-byte vector kernels
    want: every row starts on an aligned address)."""
    shape = list(shape)
    inner = shape[-1] if shape else 1
    if pad_rows and shape:
        per = max(1, alignment // element_size)
        inner = (inner + per - 1) // per * per
    stride, acc = [], 1
    for i, d in enumerate(reversed(shape)):
        stride.append(acc)
        acc *= inner if i == 0 else d
    stride.reverse()
    original = element_size * (math.prod(shape) if shape else 1)
    aligned = (acc * element_size + alignment - 1) // alignment * alignment
    return OptimizedLayout(original, aligned, aligned - original, stride)


class LayoutOptimizer:
    def __init__(self, device: DeviceInfo | None = None):
        self.device = device or DeviceInfo()

    def choose_layout(self, op, shape) -> MemoryLayout:
        op = op.kind if isinstance(op, OperationType) else op
        if op.lower().startswith("conv") and self.device.has_tensor_cores:
            return MemoryLayout.NHWC
        if len(shape) == 3:
            return MemoryLayout.BSF
        return MemoryLayout.NCHW

    @staticmethod
    def nchw_to_nhwc(x):
        return x.permute(0, 2, 3, 1).contiguous()

    @staticmethod
    def nhwc_to_nchw(x):
        return x.permute(0, 3, 1, 2).contiguous()

    def transform(self, x, src: MemoryLayout, dst: MemoryLayout):
        if src == dst:
            return x
        if (src, dst) == (MemoryLayout.NCHW, MemoryLayout.NHWC):
            return self.nchw_to_nhwc(x)
        if (src, dst) == (MemoryLayout.NHWC, MemoryLayout.NCHW):
            return self.nhwc_to_nchw(x)
        if {src, dst} == {MemoryLayout.BSF, MemoryLayout.SBF}:
            return x.transpose(0, 1).contiguous()
        raise ValueError(f"no transform {src} -> {dst}")


# =========================================================================== hardware
class HardwareBackend(enum.Enum):
    CPU = "cpu"
    CUDA = "cuda"
    ROCm = "rocm"
    Metal = "metal"
    TPU = "tpu"


@dataclass
class HardwareDevice:
    backend: HardwareBackend
    device_id: int
    name: str
    total_memory: int = 0
    compute_units: int = 0

    def is_available(self) -> bool:
        return self.backend == HardwareBackend.CPU or (self.backend == HardwareBackend.CUDA and torch.cuda.is_available())

    def torch_device(self):
        return torch.device("cuda", self.device_id) if self.backend == HardwareBackend.CUDA else torch.device("cpu")


def list_devices() -> list:
    devs = [HardwareDevice(HardwareBackend.CPU, 0, "cpu", 0, torch.get_num_threads())]
    if torch.cuda.is_available():
        for i in range(torch.cuda.device_count()):
            p = torch.cuda.get_device_properties(i)
            devs.append(HardwareDevice(HardwareBackend.CUDA, i, p.name, p.total_memory, p.multi_processor_count))
    return devs


class ElementwiseOp(enum.Enum):
    """Element-wise operations of the hardware façade (ghostflow-core/src/hardware.rs:239-247)."""
    Add = "add"
    Mul = "mul"
    ReLU = "relu"
    Sigmoid = "sigmoid"
    Tanh = "tanh"


class HardwareOps:
    """``matmul_hw / conv2d_hw / elementwise_hw`` on a chosen device; non-B200 backends raise NotImplementedError."""

    def __init__(self, device: HardwareDevice | None = None):
        self.device = device or list_devices()[-1]
        if self.device.backend not in (HardwareBackend.CPU, HardwareBackend.CUDA):
            raise NotImplementedError(f"backend {self.device.backend.value} is not built: this library targets B200")

    def _to(self, t):
        return t.to(self.device.torch_device())

    def matmul_hw(self, a, b):
        from .. import ops

        return ops.matmul(self._to(a), self._to(b))

    def conv2d_hw(self, x, w, bias=None, stride=1, padding=0):
        return torch.nn.functional.conv2d(self._to(x), self._to(w), None if bias is None else self._to(bias), stride, padding)

    def elementwise_hw(self, x, op, other=None):
        """``op``: an :class:`ElementwiseOp` or its name; Add / Mul take ``other``."""
        from .. import ops

        name = op.value if isinstance(op, ElementwiseOp) else str(op)
        if name in ("add", "mul"):
            if other is None:
                raise ValueError(f"{name} needs a second operand")
            x, other = self._to(x), self._to(other)
            return x + other if name == "add" else x * other
        return ops.unary(self._to(x), name)


# =========================================================================== sparse
class SparseTensorCOO:
    def __init__(self, indices, values, shape):
        self.t = torch.sparse_coo_tensor(torch.as_tensor(indices), torch.as_tensor(values), tuple(shape)).coalesce()

    @classmethod
    def from_dense(cls, dense, threshold: float = 0.0):
        d = getattr(dense, "data", dense) if not isinstance(dense, torch.Tensor) else dense
        mask = d.abs() > threshold
        idx = mask.nonzero().t()
        return cls(idx, d[mask], d.shape)

    @property
    def shape(self): return tuple(self.t.shape)
    def nnz(self) -> int: return self.t._nnz()
    def sparsity(self) -> float: return 1.0 - self.nnz() / max(1, math.prod(self.shape))
    def to_dense(self): return self.t.to_dense()
    def spmv(self, v): return torch.sparse.mm(self.t, torch.as_tensor(v).reshape(-1, 1)).reshape(-1)
    def spmm(self, other):
        o = other.t if isinstance(other, SparseTensorCOO) else torch.as_tensor(other)
        r = torch.sparse.mm(self.t, o)
        return SparseTensorCOO._wrap(r) if r.is_sparse else r
    def add(self, other): return SparseTensorCOO._wrap((self.t + other.t).coalesce())
    def transpose(self): return SparseTensorCOO._wrap(self.t.t().coalesce())
    def to_csr(self): return SparseTensorCSR(self.t.to_sparse_csr())
    def to_csc(self): return SparseTensorCSC(self.t.to_sparse_csc())

    @classmethod
    def _wrap(cls, t):
        o = cls.__new__(cls)
        o.t = t
        return o


class SparseTensorCSR:
    def __init__(self, t):
        self.t = t

    @classmethod
    def from_dense(cls, dense, threshold: float = 0.0):
        return SparseTensorCOO.from_dense(dense, threshold).to_csr()

    @property
    def shape(self): return tuple(self.t.shape)
    def nnz(self): return int(self.t.values().numel())
    def row_ptr(self): return self.t.crow_indices()
    def col_indices(self): return self.t.col_indices()
    def values(self): return self.t.values()
    def to_dense(self): return self.t.to_dense()
    def spmv(self, v): return (self.t @ torch.as_tensor(v).reshape(-1, 1)).reshape(-1)
    def spmm(self, dense): return self.t @ torch.as_tensor(dense)


class SparseTensorCSC:
    def __init__(self, t):
        self.t = t

    @classmethod
    def from_dense(cls, dense, threshold: float = 0.0):
        return SparseTensorCOO.from_dense(dense, threshold).to_csc()

    @property
    def shape(self): return tuple(self.t.shape)
    def nnz(self): return int(self.t.values().numel())
    def col_ptr(self): return self.t.ccol_indices()
    def row_indices(self): return self.t.row_indices()
    def values(self): return self.t.values()
    def to_dense(self): return self.t.to_dense()
    def spmv(self, v): return self.to_dense() @ torch.as_tensor(v)


# =========================================================================== metrics
class StepLogger:
    """Appends one JSON object per training step (loss, tokens/s, step ms, exposed-comm ms, peak memory, ...)."""

    def __init__(self, path: str | None = None):
        self.path, self.records = path, []
        self._t = None

    def begin_step(self):
        self._t = time.perf_counter()

    def end_step(self, step: int, loss=None, tokens: int | None = None, **extra) -> dict:
        dt = time.perf_counter() - self._t if self._t else None
        rec = {"step": step, "loss": None if loss is None else float(loss), "step_ms": None if dt is None else dt * 1e3,
               "tokens_per_s": (tokens / dt) if (tokens and dt) else None, **extra}
        if torch.cuda.is_available():
            rec["peak_mem_bytes"] = torch.cuda.max_memory_allocated()
        self.records.append(rec)
        if self.path:
            with open(self.path, "a") as f:
                f.write(json.dumps(rec) + "\n")
        return rec
