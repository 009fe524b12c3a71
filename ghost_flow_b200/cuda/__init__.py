"""Device layer with the reference's names (ghostflow-cuda/src/{lib,device,stream,memory,error}.rs):
``is_available, device_count, init, synchronize, set_device, current_device, memory_info, empty_cache, cuda_version``;
``CudaDevice`` (properties, capability predicates, ``select_best_device``), ``DeviceGuard``, ``CudaStream``,
``CudaEvent``, ``CudaTimer``, ``GpuMemoryPool`` (power-of-two size classes, ``current_usage / peak_usage``),
``CudaError``, and ``cuda.Tensor`` (the advertised ``gf.cuda.Tensor.randn(shape, device=0)``).

The reference's copies to and from the device are no-ops and its tensor read-back returns zeros
(ghostflow-cuda/src/tensor.rs:63-67,112-123); everything here moves real data through PyTorch's CUDA runtime.
"""
from __future__ import annotations

import enum

import torch

from ..tensor import Tensor as _Tensor


class CudaError(RuntimeError):
    class Kind(enum.Enum):
        NotAvailable = "cuda is not available"
        InvalidDevice = "invalid device ordinal"
        OutOfMemory = "out of memory"
        LaunchFailure = "kernel launch failed"
        InvalidValue = "invalid value"
        Unknown = "unknown error"

    def __init__(self, kind: "CudaError.Kind", detail: str = ""):
        super().__init__(f"{kind.value}{': ' + detail if detail else ''}")
        self.kind = kind


def is_available() -> bool:
    return torch.cuda.is_available()


def device_count() -> int:
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


def _require():
    if not torch.cuda.is_available():
        raise CudaError(CudaError.Kind.NotAvailable)


def init() -> None:
    _require()
    torch.cuda.init()


def cuda_version() -> tuple:
    v = torch.version.cuda or "0.0"
    a, b = v.split(".")[:2]
    return int(a), int(b)


def synchronize(device=None) -> None:
    _require()
    torch.cuda.synchronize(device)


def set_device(device_id: int) -> None:
    _require()
    if not 0 <= device_id < device_count():
        raise CudaError(CudaError.Kind.InvalidDevice, str(device_id))
    torch.cuda.set_device(device_id)


def current_device() -> int:
    _require()
    return torch.cuda.current_device()


def memory_info(device=None) -> tuple:
    """(free_bytes, total_bytes)."""
    _require()
    return torch.cuda.mem_get_info(device)


def empty_cache() -> None:
    if torch.cuda.is_available():
        torch.cuda.empty_cache()


class CudaDevice:
    def __init__(self, device_id: int = 0):
        _require()
        if not 0 <= device_id < device_count():
            raise CudaError(CudaError.Kind.InvalidDevice, str(device_id))
        self.device_id = device_id
        self.props = torch.cuda.get_device_properties(device_id)

    @property
    def name(self): return self.props.name
    @property
    def compute_capability(self): return (self.props.major, self.props.minor)
    @property
    def total_memory(self): return self.props.total_memory
    @property
    def multiprocessor_count(self): return self.props.multi_processor_count

    def memory_info(self): return torch.cuda.mem_get_info(self.device_id)
    def set_current(self): torch.cuda.set_device(self.device_id)
    def synchronize(self): torch.cuda.synchronize(self.device_id)
    def has_tensor_cores(self): return self.props.major >= 7
    def supports_bf16(self): return self.props.major >= 8
    def supports_fp8(self): return (self.props.major, self.props.minor) >= (8, 9)
    def supports_tcgen05(self): return self.props.major == 10

    def optimal_block_size(self) -> int:
        return 256

    def score(self) -> float:
        """cc * 100 + GiB, the reference's ranking (ghostflow-cuda/src/device.rs:321-350)."""
        return (self.props.major * 10 + self.props.minor) * 100 + self.props.total_memory / (1 << 30)

    def __repr__(self):
        return f"CudaDevice({self.device_id}, {self.name}, cc {self.props.major}.{self.props.minor})"


def get_all_devices():
    return [CudaDevice(i) for i in range(device_count())]


def select_best_device():
    devs = get_all_devices()
    if not devs:
        raise CudaError(CudaError.Kind.NotAvailable)
    return max(devs, key=lambda d: d.score())


class DeviceGuard:
    """RAII-style ``with DeviceGuard(1): ...``; restores the previous device on exit."""

    def __init__(self, device_id: int):
        self.device_id = device_id

    def __enter__(self):
        self.prev = current_device()
        set_device(self.device_id)
        return self

    def __exit__(self, *a):
        set_device(self.prev)
        return False


class CudaEvent:
    def __init__(self, timing: bool = True):
        _require()
        self.event = torch.cuda.Event(enable_timing=timing)

    def record(self, stream: "CudaStream | None" = None):
        self.event.record(stream.stream if stream else None)

    def synchronize(self):
        self.event.synchronize()

    def query(self) -> bool:
        return self.event.query()

    def elapsed_ms(self, end: "CudaEvent") -> float:
        return self.event.elapsed_time(end.event)


class CudaStream:
    def __init__(self, device=None, priority: int = 0, _wrap=None):
        _require()
        self.stream = _wrap if _wrap is not None else torch.cuda.Stream(device, priority=priority)

    @classmethod
    def default(cls, device=None):
        return cls(_wrap=torch.cuda.default_stream(device))

    @classmethod
    def current(cls, device=None):
        return cls(_wrap=torch.cuda.current_stream(device))

    def synchronize(self):
        self.stream.synchronize()

    def query(self) -> bool:
        return self.stream.query()

    def wait_event(self, event: CudaEvent):
        """Makes later work on this stream wait for the event on the device (the reference does a full host
        synchronise here, ghostflow-cuda/src/stream.rs:8-95)."""
        self.stream.wait_event(event.event)

    def wait_stream(self, other: "CudaStream"):
        self.stream.wait_stream(other.stream)

    def __enter__(self):
        self._ctx = torch.cuda.stream(self.stream)
        self._ctx.__enter__()
        return self

    def __exit__(self, *a):
        return self._ctx.__exit__(*a)


class CudaTimer:
    def __init__(self):
        self.e0, self.e1 = CudaEvent(), CudaEvent()

    def start(self, stream=None):
        self.e0.record(stream)

    def stop(self, stream=None):
        self.e1.record(stream)

    def elapsed_ms(self) -> float:
        self.e1.synchronize()
        return self.e0.elapsed_ms(self.e1)


class GpuMemoryPool:
    """Power-of-two size classes with free lists, on top of the device allocator."""

    def __init__(self, device=None):
        _require()
        self.device = torch.device("cuda", current_device() if device is None else device)
        self.free_lists: dict[int, list] = {}
        self.allocated: dict[int, int] = {}
        self._current = 0
        self._peak = 0
        self.hits = 0
        self.misses = 0

    @staticmethod
    def size_class(nbytes: int) -> int:
        return 1 << max(8, (max(1, nbytes) - 1).bit_length())

    def allocate(self, nbytes: int) -> torch.Tensor:
        sc = self.size_class(nbytes)
        lst = self.free_lists.get(sc)
        if lst:
            buf = lst.pop()
            self.hits += 1
        else:
            try:
                buf = torch.empty(sc, dtype=torch.uint8, device=self.device)
            except torch.cuda.OutOfMemoryError as e:
                raise CudaError(CudaError.Kind.OutOfMemory, str(e)) from e
            self.misses += 1
        self.allocated[buf.data_ptr()] = sc
        self._current += sc
        self._peak = max(self._peak, self._current)
        return buf

    def free(self, buf: torch.Tensor):
        sc = self.allocated.pop(buf.data_ptr(), None)
        if sc is None:
            raise CudaError(CudaError.Kind.InvalidValue, "buffer does not belong to this pool")
        self.free_lists.setdefault(sc, []).append(buf)
        self._current -= sc

    def clear(self):
        self.free_lists.clear()
        torch.cuda.empty_cache()

    def current_usage(self) -> int:
        return self._current

    def peak_usage(self) -> int:
        return self._peak


_GLOBAL_POOL = None


def get_global_gpu_pool() -> GpuMemoryPool:
    global _GLOBAL_POOL
    if _GLOBAL_POOL is None:
        _GLOBAL_POOL = GpuMemoryPool()
    return _GLOBAL_POOL


class Tensor(_Tensor):
    """``gf.cuda.Tensor.randn(shape, device=0)`` and friends: a :class:`ghost_flow_b200.Tensor` living on a GPU."""

    @staticmethod
    def _dev(device):
        _require()
        return torch.device("cuda", device if isinstance(device, int) else torch.device(device).index or 0)

    @staticmethod
    def randn(*shape, device=0, dtype=None):
        return _Tensor.randn(*shape, device=Tensor._dev(device), dtype=dtype)

    @staticmethod
    def rand(*shape, device=0, dtype=None):
        return _Tensor.rand(*shape, device=Tensor._dev(device), dtype=dtype)

    @staticmethod
    def zeros(*shape, device=0, dtype=None):
        return _Tensor.zeros(*shape, device=Tensor._dev(device), dtype=dtype)

    @staticmethod
    def ones(*shape, device=0, dtype=None):
        return _Tensor.ones(*shape, device=Tensor._dev(device), dtype=dtype)

    @staticmethod
    def from_tensor(t, device=0):
        return _Tensor(getattr(t, "data", t).to(Tensor._dev(device)))


# --------------------------------------------------------------------------------------------- result / launch types
CudaResult = object        # functions here return values or raise CudaError; the alias keeps the reference's name


def check_cuda_error(code: int = 0, what: str = "") -> None:
    """Raises :class:`CudaError` for a non-zero runtime code (and for a pending asynchronous error)."""
    if code != 0:
        raise CudaError(CudaError.Kind.Unknown, f"{what} (code {code})")
    if torch.cuda.is_available():
        torch.cuda.synchronize()


class LaunchConfig:
    """grid / block / dynamic shared memory of a launch, with the reference's helpers
    (ghostflow-cuda/src/kernels/mod.rs:8-41)."""

    def __init__(self, grid=(1, 1, 1), block=(256, 1, 1), shared: int = 0):
        self.grid, self.block, self.shared = tuple(grid), tuple(block), shared

    @classmethod
    def for_elements(cls, n: int, block: int = 256):
        return cls(((n + block - 1) // block, 1, 1), (block, 1, 1), 0)

    @classmethod
    def for_2d(cls, rows: int, cols: int, tile: int = 16):
        return cls(((cols + tile - 1) // tile, (rows + tile - 1) // tile, 1), (tile, tile, 1), 0)

    @classmethod
    def persistent(cls, threads: int = 192, shared: int = 0, device: int = 0):
        """One CTA per SM: the shape of this library's GEMM / attention kernels."""
        sms = torch.cuda.get_device_properties(device).multi_processor_count if torch.cuda.is_available() else 148
        return cls((sms, 1, 1), (threads, 1, 1), shared)


# The 17 kernel names of the reference's intended surface (kernels/mod.rs:47-110) and the entry points of this
# library that implement them.
KERNELS = {
    "add": "gf_binary", "mul": "gf_binary", "relu": "gf_unary", "gelu": "gf_unary", "sigmoid": "gf_unary",
    "matmul": "gf_gemm_bf16", "matmul_tiled": "gf_gemm_bf16", "matmul_tensor_core": "gf_gemm_bf16",
    "flash_attention_forward": "gf_flash_attn_fwd3", "flash_attention_backward": "gf_flash_attn_bwd2",
    "sum_reduce": "gf_reduce", "max_reduce": "gf_reduce", "softmax": "gf_softmax_rows",
    "cross_entropy": "gf_xent_fused", "layer_norm": "gf_layernorm_fwd", "rms_norm": "gf_rmsnorm_fwd",
    "batch_norm": "gf_batchnorm_train",
}


class GpuTensor:
    """fp32 device buffer with real copies in both directions (ghostflow-cuda/src/memory.rs:148-251)."""

    def __init__(self, shape, device: int = 0):
        _require()
        self.shape = tuple(shape)
        self.t = torch.empty(self.shape, dtype=torch.float32, device=torch.device("cuda", device))

    @classmethod
    def from_cpu(cls, data, shape=None, device: int = 0):
        src = torch.as_tensor(data, dtype=torch.float32)
        g = cls(tuple(shape) if shape is not None else tuple(src.shape), device)
        g.copy_from_cpu(src)
        return g

    def copy_from_cpu(self, data):
        self.t.copy_(torch.as_tensor(data, dtype=torch.float32).reshape(self.shape), non_blocking=False)

    def copy_to_cpu(self) -> torch.Tensor:
        return self.t.detach().cpu()

    def numel(self) -> int:
        return self.t.numel()

    def size_bytes(self) -> int:
        return self.t.numel() * 4


class CudaTensor:
    """Device tensor with the reference's method set (ghostflow-cuda/src/tensor.rs). The reference elides every
    memcpy and falls back to the CPU for most ops; here data lives on the GPU and ops run there (matmul on the
    tcgen05 GEMM kernel when the operands are bf16)."""

    def __init__(self, data, device: int = 0):
        _require()
        src = getattr(data, "data", data)
        self.device_id = device
        self.t = torch.as_tensor(src).to(torch.device("cuda", device))

    @classmethod
    def from_tensor(cls, t, device: int = 0): return cls(t, device)
    @classmethod
    def zeros(cls, shape, device=0, dtype=torch.float32): return cls(torch.zeros(*shape, dtype=dtype), device)
    @classmethod
    def ones(cls, shape, device=0, dtype=torch.float32): return cls(torch.ones(*shape, dtype=dtype), device)
    @classmethod
    def full(cls, shape, value, device=0, dtype=torch.float32): return cls(torch.full(tuple(shape), value, dtype=dtype), device)

    @property
    def shape(self): return tuple(self.t.shape)
    @property
    def strides(self): return tuple(self.t.stride())
    @property
    def dtype(self): return self.t.dtype
    @property
    def size_bytes(self): return self.t.numel() * self.t.element_size()
    @property
    def ptr(self): return self.t.data_ptr()

    def _w(self, t):
        c = CudaTensor.__new__(CudaTensor)
        c.device_id, c.t = self.device_id, t
        return c

    def to_tensor(self): return _Tensor(self.t.detach().cpu())
    def clone(self): return self._w(self.t.clone())
    def reshape(self, shape): return self._w(self.t.reshape(tuple(shape)))
    def transpose(self, d0=0, d1=1): return self._w(self.t.transpose(d0, d1))
    def add(self, o): return self._w(self.t + o.t)
    def sub(self, o): return self._w(self.t - o.t)
    def mul(self, o): return self._w(self.t * o.t)
    def mul_scalar(self, s): return self._w(self.t * s)
    def relu(self): return self._w(torch.relu(self.t))
    def dot(self, o): return float((self.t.flatten().float() * o.t.flatten().float()).sum())
    def norm(self): return float(self.t.float().norm())

    def matmul(self, o):
        from ..ops.gemm import matmul as gf_matmul
        return self._w(gf_matmul(self.t, o.t))


class CuBlas:
    """BLAS-shaped entry points (ghostflow-cuda/src/blas.rs). ``sgemm`` on bf16 operands runs this library's
    tcgen05 GEMM; fp32 operands go through the vendor library, which is the reference's own arrangement."""

    def __init__(self, device: int = 0):
        _require()
        self.device = torch.device("cuda", device)

    def sgemm(self, a: torch.Tensor, b: torch.Tensor, alpha: float = 1.0, beta: float = 0.0, c: torch.Tensor | None = None):
        from ..ops.gemm import matmul as gf_matmul
        y = gf_matmul(a, b)  # bf16: tcgen05 kernel; fp32: the same kernel over hi/lo bf16 splits
        y = y if alpha == 1.0 else y * alpha
        return y if c is None or beta == 0.0 else y + beta * c

    def saxpy(self, alpha: float, x: torch.Tensor, y: torch.Tensor): return y.add_(x, alpha=alpha)
    def sscal(self, alpha: float, x: torch.Tensor): return x.mul_(alpha)
    def sdot(self, x, y): return float((x.float() * y.float()).sum())
    def snrm2(self, x): return float(x.float().norm())

    def matmul(self, a: CudaTensor, b: CudaTensor) -> CudaTensor:
        return a.matmul(b)
