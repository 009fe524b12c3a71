"""Core value types with the reference's names: ``Shape`` / ``Strides`` (numpy broadcasting, contiguity, offsets),
device markers, the error type, the ``Serializable`` protocol and the host layout helper.

Reference: ghostflow-core/src/shape.rs:50-156 (broadcast, default strides, ``is_contiguous``), device.rs:6-45
(``Device`` trait, ``Cpu``, ``Cuda{device_id}``), error.rs:7-52 (``GhostError``, 15 variants), dtype.rs:33-40
(``TensorElement``), serialize.rs:203-220 (``Serializable``), memory.rs:105-154 (``MemoryLayoutOptimizer``, 64-byte
alignment). Tensors themselves are ``torch.Tensor`` wrapped by :class:`ghost_flow_b200.Tensor`; these types are the
small value objects around them."""
from __future__ import annotations

import enum
from typing import Iterable, Sequence

import torch


class GhostError(Exception):
    """One exception type with a ``kind`` (the reference's enum variants)."""

    class Kind(enum.Enum):
        ShapeMismatch = "shape mismatch"
        InvalidShape = "invalid shape"
        DimOutOfBounds = "dimension out of bounds"
        IndexOutOfBounds = "index out of bounds"
        DTypeMismatch = "dtype mismatch"
        DeviceMismatch = "device mismatch"
        DeviceError = "device error"
        BroadcastError = "shapes cannot be broadcast"
        InvalidOperation = "invalid operation"
        InvalidFormat = "invalid format"
        InvalidParameter = "invalid parameter"
        NotTrained = "model is not trained"
        NotImplemented = "not implemented"
        IOError = "i/o error"
        OutOfMemory = "out of memory"

    def __init__(self, kind: "GhostError.Kind", detail: str = ""):
        super().__init__(f"{kind.value}{': ' + detail if detail else ''}")
        self.kind = kind


class Strides(tuple):
    """Element strides, innermost last."""

    def __new__(cls, values: Iterable[int] = ()):
        return super().__new__(cls, (int(v) for v in values))


class Shape(tuple):
    """Dimension sizes with numpy-style helpers."""

    def __new__(cls, dims: Iterable[int] = ()):
        dims = tuple(int(d) for d in dims)
        if any(d < 0 for d in dims):
            raise GhostError(GhostError.Kind.InvalidShape, str(dims))
        return super().__new__(cls, dims)

    @property
    def ndim(self) -> int:
        return len(self)

    def dims(self):
        return tuple(self)

    def numel(self) -> int:
        n = 1
        for d in self:
            n *= d
        return n

    def default_strides(self) -> Strides:
        s, acc = [], 1
        for d in reversed(self):
            s.append(acc)
            acc *= d
        return Strides(reversed(s))

    def is_contiguous(self, strides: Sequence[int]) -> bool:
        expect = 1
        for d, st in zip(reversed(self), reversed(tuple(strides))):
            if d != 1 and st != expect:
                return False
            expect *= d
        return True

    def offset(self, index: Sequence[int], strides: Sequence[int] | None = None) -> int:
        strides = strides if strides is not None else self.default_strides()
        if len(index) != len(self):
            raise GhostError(GhostError.Kind.DimOutOfBounds, f"{len(index)} indices for {len(self)} dims")
        off = 0
        for i, d, s in zip(index, self, strides):
            if not 0 <= i < d:
                raise GhostError(GhostError.Kind.IndexOutOfBounds, f"{i} in dim of size {d}")
            off += i * s
        return off

    def broadcast_with(self, other: "Shape") -> "Shape":
        a, b = tuple(self), tuple(other)
        n = max(len(a), len(b))
        a, b = (1,) * (n - len(a)) + a, (1,) * (n - len(b)) + b
        out = []
        for x, y in zip(a, b):
            if x != y and x != 1 and y != 1:
                raise GhostError(GhostError.Kind.BroadcastError, f"{tuple(self)} vs {tuple(other)}")
            out.append(max(x, y))
        return Shape(out)

    def transpose(self, d0: int, d1: int) -> "Shape":
        l = list(self)
        l[d0], l[d1] = l[d1], l[d0]
        return Shape(l)

    def squeeze(self) -> "Shape":
        return Shape(d for d in self if d != 1)


class Device:
    """Device marker (``Cpu()`` / ``Cuda(device_id)``); ``torch_device()`` gives the torch object."""
    name = "device"

    def torch_device(self) -> torch.device:
        raise NotImplementedError

    def __eq__(self, other):
        return isinstance(other, Device) and self.torch_device() == other.torch_device()

    def __hash__(self):
        return hash(str(self.torch_device()))

    def __repr__(self):
        return f"{type(self).__name__}({self.torch_device()})"


class Cpu(Device):
    name = "cpu"

    def torch_device(self):
        return torch.device("cpu")


class Cuda(Device):
    name = "cuda"

    def __init__(self, device_id: int = 0):
        self.device_id = device_id

    def torch_device(self):
        return torch.device("cuda", self.device_id)


# Element types a tensor can be built from (the reference has no f16 / bf16 element type; here they exist).
TensorElement = (float, int, bool)
StateDict = dict


class Storage:
    """Flat typed buffer behind a tensor (ghostflow-core/src/storage.rs:8-120): a 1-D torch tensor plus a
    readers-writer lock; ``read()`` / ``write()`` are the guards (context managers that yield the buffer)."""

    def __init__(self, dtype=torch.float32, length: int = 0, device="cpu"):
        import threading

        self.data = torch.zeros(length, dtype=dtype, device=device)
        self._cond = threading.Condition()
        self._readers = 0
        self._writing = False

    @classmethod
    def from_slice(cls, values, dtype=torch.float32, device="cpu"):
        s = cls(dtype, 0, device)
        s.data = torch.as_tensor(values, dtype=dtype, device=device).reshape(-1).clone()
        return s

    def __len__(self):
        return self.data.numel()

    def len(self):
        return self.data.numel()

    def is_empty(self):
        return self.data.numel() == 0

    @property
    def dtype(self):
        return self.data.dtype

    def read(self):
        return StorageReadGuard(self)

    def write(self):
        return StorageWriteGuard(self)


class StorageReadGuard:
    """Shared access: any number of readers, no writer."""

    def __init__(self, storage: Storage):
        self.s = storage

    def __enter__(self):
        with self.s._cond:
            while self.s._writing:
                self.s._cond.wait()
            self.s._readers += 1
        return self.s.data

    def __exit__(self, *exc):
        with self.s._cond:
            self.s._readers -= 1
            self.s._cond.notify_all()
        return False


class StorageWriteGuard:
    """Exclusive access."""

    def __init__(self, storage: Storage):
        self.s = storage

    def __enter__(self):
        with self.s._cond:
            while self.s._writing or self.s._readers:
                self.s._cond.wait()
            self.s._writing = True
        return self.s.data

    def __exit__(self, *exc):
        with self.s._cond:
            self.s._writing = False
            self.s._cond.notify_all()
        return False


class Serializable:
    """Mix-in: anything with ``state_dict()`` / ``load_state_dict()`` gains ``save(path)`` / ``load(path)`` in the
    GHOSTFLW format (or GFCP / safetensors by extension or ``fmt``)."""

    def state_dict(self) -> dict:
        raise NotImplementedError

    def load_state_dict(self, state: dict):
        raise NotImplementedError

    def save(self, path, fmt: str | None = None):
        from . import io as gf_io
        fmt = fmt or ("safetensors" if str(path).endswith(".safetensors") else "ghostflw")
        gf_io.save_state_dict({k: getattr(v, "data", v) for k, v in self.state_dict().items()}, path, fmt)

    def load(self, path):
        from . import io as gf_io
        self.load_state_dict(gf_io.load_state_dict(path))
        return self


class MemoryLayoutOptimizer:
    """Sizes and offsets for packing tensors into one allocation with every tensor aligned to ``alignment`` bytes."""

    def __init__(self, alignment: int = 64):
        self.alignment = alignment

    def align(self, nbytes: int) -> int:
        a = self.alignment
        return (nbytes + a - 1) // a * a

    def plan(self, sizes: Sequence[int]):
        """Returns (offsets, total bytes)."""
        offs, cur = [], 0
        for s in sizes:
            offs.append(cur)
            cur += self.align(s)
        return offs, cur

    def pack(self, tensors: Sequence[torch.Tensor]):
        """One flat uint8 buffer holding all tensors at aligned offsets, plus views into it."""
        offs, total = self.plan([t.numel() * t.element_size() for t in tensors])
        dev = tensors[0].device if tensors else "cpu"
        buf = torch.zeros(total, dtype=torch.uint8, device=dev)
        views = []
        for t, o in zip(tensors, offs):
            n = t.numel() * t.element_size()
            v = buf[o:o + n].view(t.dtype).view(t.shape)
            v.copy_(t)
            views.append(v)
        return buf, views
