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
