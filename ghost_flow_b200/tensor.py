"""``ghost_flow.Tensor``: the user-facing tensor with autograd, over ``torch.Tensor`` storage.

Surface = what the reference's Python binding really exposes (ghost-flow-py/src/lib.rs:20-170:
``Tensor(data, shape)``, ``zeros/ones/randn/rand``, ``shape/ndim/size``, ``matmul``, ``+ - * @``,
``transpose``, ``reshape``, ``relu/sigmoid/gelu``, ``softmax(dim)``, ``sum/mean`` -> 0-d tensor, flat
``tolist()``) plus what its README advertises and the Rust core has (README.md:217-283;
ghostflow-core/src/tensor.rs:38-340, ops/arithmetic.rs, ops/reduction.rs): scalars in arithmetic,
``backward()``, ``grad``, ``item()``, ``** 2``, views, reductions along a dim, creation helpers.
"""
from __future__ import annotations

import math
from typing import Iterable, Sequence

import torch

from .dtype import DType, to_torch_dtype
from . import ops as _ops
from .ops import elementwise as _ew

_DEFAULT_DEVICE = torch.device("cpu")


def set_default_device(device) -> None:
    global _DEFAULT_DEVICE
    _DEFAULT_DEVICE = torch.device(device)


def get_default_device() -> torch.device:
    return _DEFAULT_DEVICE


def manual_seed(seed: int) -> None:
    """Seeds every generator (the reference has no seed API: ghostflow-core/src/tensor.rs:94,105)."""
    torch.manual_seed(seed)
    if torch.cuda.is_available():
        torch.cuda.manual_seed_all(seed)


def _unwrap(x):
    return x.data if isinstance(x, Tensor) else x


def _shape_arg(shape) -> tuple:
    if len(shape) == 1 and isinstance(shape[0], (list, tuple, torch.Size)):
        return tuple(shape[0])
    return tuple(shape)


class Tensor:
    """A dense tensor. ``Tensor(data, shape)`` takes a flat (or nested) list like the reference."""

    __slots__ = ("data",)
    __array_priority__ = 100

    def __init__(self, data, shape: Sequence[int] | None = None, dtype=None, device=None, requires_grad=False):
        if isinstance(data, Tensor):
            t = data.data
        elif isinstance(data, torch.Tensor):
            t = data
        else:
            t = torch.tensor(data, dtype=to_torch_dtype(dtype) if dtype is not None else torch.float32,
                             device=device or _DEFAULT_DEVICE)
        if shape is not None:
            n = 1
            for s in shape:
                n *= s
            if n != t.numel():
                raise ValueError(f"shape {list(shape)} does not match {t.numel()} elements")
            t = t.reshape(tuple(shape))
        if dtype is not None and isinstance(data, (Tensor, torch.Tensor)):
            t = t.to(to_torch_dtype(dtype))
        if device is not None and isinstance(data, (Tensor, torch.Tensor)):
            t = t.to(device)
        if requires_grad:
            t = t.detach().requires_grad_(True)
        self.data = t

    # ------------------------------------------------------------------ creation
    @staticmethod
    def _make(fn, shape, dtype, device, requires_grad, **kw):
        t = fn(_shape_arg(shape), dtype=to_torch_dtype(dtype) if dtype is not None else torch.float32,
               device=device or _DEFAULT_DEVICE, **kw)
        return Tensor(t.requires_grad_(requires_grad))

    @staticmethod
    def zeros(*shape, dtype=None, device=None, requires_grad=False):
        return Tensor._make(torch.zeros, shape, dtype, device, requires_grad)

    @staticmethod
    def ones(*shape, dtype=None, device=None, requires_grad=False):
        return Tensor._make(torch.ones, shape, dtype, device, requires_grad)

    @staticmethod
    def full(shape, value, dtype=None, device=None, requires_grad=False):
        return Tensor._make(torch.full, (shape,), dtype, device, requires_grad, fill_value=value)

    @staticmethod
    def randn(*shape, dtype=None, device=None, requires_grad=False):
        return Tensor._make(torch.randn, shape, dtype, device, requires_grad)

    @staticmethod
    def rand(*shape, dtype=None, device=None, requires_grad=False):
        return Tensor._make(torch.rand, shape, dtype, device, requires_grad)

    @staticmethod
    def eye(n, dtype=None, device=None):
        return Tensor(torch.eye(n, dtype=to_torch_dtype(dtype) if dtype else torch.float32,
                                device=device or _DEFAULT_DEVICE))

    @staticmethod
    def arange(start, end=None, step=1, dtype=None, device=None):
        if end is None:
            start, end = 0, start
        return Tensor(torch.arange(start, end, step, dtype=to_torch_dtype(dtype) if dtype else torch.float32,
                                   device=device or _DEFAULT_DEVICE))

    @staticmethod
    def linspace(start, end, steps, dtype=None, device=None):
        return Tensor(torch.linspace(start, end, steps, dtype=to_torch_dtype(dtype) if dtype else torch.float32,
                                     device=device or _DEFAULT_DEVICE))

    @staticmethod
    def from_slice(data: Iterable[float], shape: Sequence[int]):
        return Tensor(list(data), list(shape))

    @staticmethod
    def from_numpy(arr):
        return Tensor(torch.from_numpy(arr))

    # ------------------------------------------------------------------ properties
    @property
    def shape(self):
        return list(self.data.shape)

    def dims(self):
        return list(self.data.shape)

    @property
    def ndim(self):
        return self.data.dim()

    @property
    def size(self):
        return self.data.numel()

    def numel(self):
        return self.data.numel()

    @property
    def dtype(self):
        return DType.from_torch(self.data.dtype)

    @property
    def device(self):
        return self.data.device

    @property
    def requires_grad(self):
        return self.data.requires_grad

    @requires_grad.setter
    def requires_grad(self, v):
        self.data.requires_grad_(v)

    def requires_grad_(self, v=True):
        self.data.requires_grad_(v)
        return self

    @property
    def grad(self):
        g = self.data.grad
        return Tensor(g) if g is not None else None

    def set_grad(self, g):
        self.data.grad = _unwrap(g)

    def zero_grad(self):
        self.data.grad = None

    def is_contiguous(self):
        return self.data.is_contiguous()

    # ------------------------------------------------------------------ conversion
    def tolist(self):
        """Flat list of floats in row-major order (ghost-flow-py/src/lib.rs: ``tolist``)."""
        return self.data.detach().reshape(-1).to(torch.float32).cpu().tolist()

    def to_nested_list(self):
        return self.data.detach().cpu().tolist()

    def data_f32(self):
        return self.tolist()

    def item(self):
        return self.data.item()

    def numpy(self):
        return self.data.detach().to(torch.float32).cpu().numpy() if self.data.dtype == torch.bfloat16 \
            else self.data.detach().cpu().numpy()

    def torch(self) -> torch.Tensor:
        return self.data

    def to(self, *args, **kw):
        args = tuple(to_torch_dtype(a) if isinstance(a, (DType, str)) and not _is_device(a) else a for a in args)
        return Tensor(self.data.to(*args, **kw))

    def cuda(self, device=0):
        return Tensor(self.data.cuda(device))

    def cpu(self):
        return Tensor(self.data.cpu())

    def float(self):
        return Tensor(self.data.float())

    def bfloat16(self):
        return Tensor(self.data.bfloat16())

    def half(self):
        return Tensor(self.data.half())

    def detach(self):
        return Tensor(self.data.detach())

    def clone(self):
        return Tensor(self.data.clone())

    deep_clone = clone

    # ------------------------------------------------------------------ autograd
    def backward(self, grad=None, retain_graph=False):
        """Reverse-mode differentiation from this tensor (scalar unless ``grad`` is given).
        The reference's ``backward`` only asserts a scalar and returns
        (ghostflow-autograd/src/backward.rs:11-25); this one runs the graph."""
        self.data.backward(_unwrap(grad), retain_graph=retain_graph)

    # ------------------------------------------------------------------ arithmetic
    def _bin(self, other, fn):
        return Tensor(fn(self.data, _unwrap(other)))

    def _ew(self, other, op):
        """add / sub / mul of two dense same-shape CUDA tensors runs the library's element-wise kernel."""
        return Tensor(_ew.binary(self.data, _unwrap(other), op))

    def __add__(self, o): return self._ew(o, "add")
    def __radd__(self, o): return self._bin(o, torch.add)
    def __sub__(self, o): return self._ew(o, "sub")
    def __rsub__(self, o): return Tensor(torch.sub(_as_t(o, self.data), self.data))
    def __mul__(self, o): return self._ew(o, "mul")
    def __rmul__(self, o): return self._bin(o, torch.mul)
    def __truediv__(self, o): return self._bin(o, torch.div)
    def __rtruediv__(self, o): return Tensor(torch.div(_as_t(o, self.data), self.data))
    def __pow__(self, o): return self._bin(o, torch.pow)
    def __neg__(self): return Tensor(-self.data)
    def __matmul__(self, o): return self.matmul(o)
    def __getitem__(self, idx): return Tensor(self.data[_unwrap(idx)])
    def __len__(self): return self.data.shape[0]

    add = __add__
    sub = __sub__
    mul = __mul__
    div = __truediv__

    def add_scalar(self, s): return Tensor(self.data + s)
    def mul_scalar(self, s): return Tensor(self.data * s)
    def neg(self): return Tensor(-self.data)
    def abs(self): return Tensor(self.data.abs())
    def pow(self, e): return Tensor(self.data.pow(_unwrap(e)))
    def sqrt(self): return Tensor(self.data.sqrt())
    def exp(self): return Tensor(self.data.exp())
    def log(self): return Tensor(self.data.log())
    def clamp(self, lo=None, hi=None): return Tensor(self.data.clamp(lo, hi))

    def matmul(self, other):
        """Matrix product; 2-D bf16 CUDA operands run the tcgen05 GEMM kernel."""
        return Tensor(_ops.matmul(self.data, _unwrap(other)))

    def dot(self, o): return Tensor(torch.dot(self.data.reshape(-1), _unwrap(o).reshape(-1)))
    def outer(self, o): return Tensor(torch.outer(self.data, _unwrap(o)))
    def mv(self, o): return Tensor(torch.mv(self.data, _unwrap(o)))
    def bmm(self, o): return Tensor(torch.bmm(self.data, _unwrap(o)))
    def trace(self): return Tensor(torch.trace(self.data))
    def diag(self): return Tensor(torch.diag(self.data))

    # ------------------------------------------------------------------ views
    def reshape(self, *shape): return Tensor(self.data.reshape(_shape_arg(shape)))
    view = reshape
    def flatten(self): return Tensor(self.data.reshape(-1))
    def transpose(self, d0, d1): return Tensor(self.data.transpose(d0, d1))
    def t(self): return Tensor(self.data.transpose(-1, -2) if self.data.dim() >= 2 else self.data)
    def permute(self, *dims): return Tensor(self.data.permute(_shape_arg(dims)))
    def squeeze(self, dim=None): return Tensor(self.data.squeeze() if dim is None else self.data.squeeze(dim))
    def unsqueeze(self, dim): return Tensor(self.data.unsqueeze(dim))
    def contiguous(self): return Tensor(self.data.contiguous())

    # ------------------------------------------------------------------ activations
    def relu(self): return Tensor(_ew.unary_any(self.data, "relu"))
    def sigmoid(self): return Tensor(_ew.unary_any(self.data, "sigmoid"))
    def tanh(self): return Tensor(_ew.unary_any(self.data, "tanh"))
    def gelu(self): return Tensor(_ew.unary_any(self.data, "gelu"))
    def silu(self): return Tensor(_ew.unary_any(self.data, "silu"))
    def leaky_relu(self, slope=0.01): return Tensor(torch.nn.functional.leaky_relu(self.data, slope))
    def elu(self, alpha=1.0): return Tensor(torch.nn.functional.elu(self.data, alpha))
    def selu(self): return Tensor(torch.selu(self.data))
    def mish(self): return Tensor(torch.nn.functional.mish(self.data))
    def softplus(self, beta=1.0, threshold=20.0): return Tensor(torch.nn.functional.softplus(self.data, beta, threshold))
    def softsign(self): return Tensor(torch.nn.functional.softsign(self.data))
    def hardtanh(self, lo=-1.0, hi=1.0): return Tensor(torch.nn.functional.hardtanh(self.data, lo, hi))
    def hardsigmoid(self): return Tensor(torch.nn.functional.hardsigmoid(self.data))
    def hardswish(self): return Tensor(torch.nn.functional.hardswish(self.data))
    def softmax(self, dim=-1):
        if dim in (-1, self.data.dim() - 1) and self.data.shape[-1] >= 32:
            return Tensor(_ew.softmax_rows(self.data))
        return Tensor(torch.softmax(self.data, dim))

    def log_softmax(self, dim=-1):
        if dim in (-1, self.data.dim() - 1) and self.data.shape[-1] >= 32:
            return Tensor(_ew.softmax_rows(self.data, log=True))
        return Tensor(torch.log_softmax(self.data, dim))

    # ------------------------------------------------------------------ reductions
    def _full_reduce(self, mode):
        d = self.data
        if d.is_cuda and d.is_floating_point():
            return Tensor(_ew.reduce_all(d, mode).to(d.dtype))
        return Tensor(d.sum() if mode == "sum" else d.max())

    def sum(self): return self._full_reduce("sum")
    def mean(self): return Tensor(self.data.mean())
    def max(self): return self._full_reduce("max")
    def min(self): return Tensor(self.data.min())
    def prod(self): return Tensor(self.data.prod())
    def var(self, unbiased=False): return Tensor(self.data.var(unbiased=unbiased))
    def std(self, unbiased=False): return Tensor(self.data.std(unbiased=unbiased))
    def norm(self): return Tensor(self.data.norm())
    def norm_l1(self): return Tensor(self.data.abs().sum())
    # indices come back as float tensors, like ghostflow-core/src/ops/reduction.rs:89-96
    def argmax(self, dim=None): return Tensor(self.data.argmax(dim).to(torch.float32))
    def argmin(self, dim=None): return Tensor(self.data.argmin(dim).to(torch.float32))
    def sum_dim(self, dim, keepdim=False): return Tensor(self.data.sum(dim, keepdim=keepdim))
    def mean_dim(self, dim, keepdim=False): return Tensor(self.data.mean(dim, keepdim=keepdim))
    def max_dim(self, dim, keepdim=False): return Tensor(self.data.max(dim, keepdim=keepdim).values)
    def min_dim(self, dim, keepdim=False): return Tensor(self.data.min(dim, keepdim=keepdim).values)
    def var_dim(self, dim, keepdim=False): return Tensor(self.data.var(dim, unbiased=False, keepdim=keepdim))

    def __repr__(self):
        return f"Tensor(shape={self.shape}, dtype={self.data.dtype}, device={self.data.device})"

    def __eq__(self, other):
        return Tensor(self.data == _unwrap(other))

    __hash__ = None


def _as_t(o, like):
    return o if isinstance(o, torch.Tensor) else torch.as_tensor(o, dtype=like.dtype, device=like.device)


def _is_device(a) -> bool:
    if isinstance(a, torch.device):
        return True
    return isinstance(a, str) and (a.startswith("cuda") or a == "cpu")


def zeros(*shape, **kw): return Tensor.zeros(*shape, **kw)
def ones(*shape, **kw): return Tensor.ones(*shape, **kw)
def randn(*shape, **kw): return Tensor.randn(*shape, **kw)
def rand(*shape, **kw): return Tensor.rand(*shape, **kw)
def tensor(data, **kw): return Tensor(data, **kw)


class no_grad(torch.no_grad):
    """Disables graph recording (the reference's ``no_grad`` is an empty stub: ghostflow-autograd/src/lib.rs:14-21)."""


class enable_grad(torch.enable_grad):
    pass
