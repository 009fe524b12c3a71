"""The reference's autograd surface, working: a gradient tape, ``backward``, closed-form gradient functions, and a
dynamic graph with ``with_grad`` / ``no_grad`` contexts.

Reference: ghostflow-autograd/src/tape.rs:5-121 (thread-local ``GradTape`` of ``RecordedOp``s that nothing records
into), backward.rs:11-25 (``backward`` is a no-op) and :28-191 (``grad_fns``, correct closed forms),
dynamic_graph.rs (nodes are stored with ``backward_fn: None`` so gradients never flow). Differentiation itself is
PyTorch autograd; the tape here records every op that goes through it (name, inputs, output, backward closure) and
can replay gradients on its own, which is what the tests check against torch."""
from __future__ import annotations

import contextlib
import threading
from dataclasses import dataclass, field
from typing import Callable

import torch

from .tensor import Tensor, _unwrap


@dataclass
class RecordedOp:
    op_name: str
    input_ids: list
    output_id: int
    backward_fn: Callable | None = None


class GradTape:
    """Records operations; ``gradient(output, inputs)`` walks the tape backwards through the recorded closures."""

    def __init__(self):
        self.operations: list[RecordedOp] = []
        self.enabled = True
        self._values: dict[int, torch.Tensor] = {}

    def record_op(self, op_name, inputs, output, backward_fn=None):
        if not self.enabled:
            return
        for t in list(inputs) + [output]:
            self._values[id(t)] = t
        self.operations.append(RecordedOp(op_name, [id(t) for t in inputs], id(output), backward_fn))

    def gradient(self, output, inputs, grad_output=None):
        grads = {id(output): torch.ones_like(output) if grad_output is None else grad_output}
        for op in reversed(self.operations):
            g = grads.get(op.output_id)
            if g is None or op.backward_fn is None:
                continue
            for iid, gi in zip(op.input_ids, op.backward_fn(g)):
                if gi is not None:
                    grads[iid] = grads[iid] + gi if iid in grads else gi
        return [grads.get(id(t)) for t in inputs]

    def clear(self):
        self.operations.clear()
        self._values.clear()


_LOCAL = threading.local()


def current_tape() -> GradTape | None:
    return getattr(_LOCAL, "tape", None)


def is_recording() -> bool:
    t = current_tape()
    return t is not None and t.enabled


def record_op(op_name, inputs, output, backward_fn=None):
    t = current_tape()
    if t is not None:
        t.record_op(op_name, inputs, output, backward_fn)


class GradTapeContext:
    """``with GradTapeContext() as tape: ...`` installs a tape for the thread and restores the previous one."""

    def __enter__(self):
        self._prev = current_tape()
        _LOCAL.tape = GradTape()
        return _LOCAL.tape

    def __exit__(self, *a):
        _LOCAL.tape = self._prev
        return False


def backward(t, grad=None, retain_graph=False):
    """Back-propagates from a :class:`Tensor` or torch tensor through torch autograd."""
    x = _unwrap(t)
    x.backward(_unwrap(grad) if grad is not None else None, retain_graph=retain_graph)


class grad_fns:
    """Closed-form gradients on raw tensors (the reference's slice functions), usable as oracle formulas."""

    @staticmethod
    def add_backward(g): return g, g
    @staticmethod
    def mul_backward(g, a, b): return g * b, g * a
    @staticmethod
    def relu_backward(g, x): return g * (x > 0).to(g.dtype)
    @staticmethod
    def sigmoid_backward(g, y): return g * y * (1 - y)
    @staticmethod
    def tanh_backward(g, y): return g * (1 - y * y)
    @staticmethod
    def exp_backward(g, y): return g * y
    @staticmethod
    def log_backward(g, x): return g / x
    @staticmethod
    def pow_backward(g, x, p): return g * p * x.pow(p - 1)
    @staticmethod
    def matmul_backward(g, a, b): return g @ b.transpose(-1, -2), a.transpose(-1, -2) @ g

    @staticmethod
    def softmax_cross_entropy_backward(logits, targets):
        p = torch.softmax(logits.float(), -1)
        p[torch.arange(len(targets)), targets] -= 1
        return p / len(targets)


# ------------------------------------------------------------------ dynamic graph
class DynamicContext:
    _grad = threading.local()

    @classmethod
    def grad_enabled(cls) -> bool:
        return getattr(cls._grad, "on", True)

    @classmethod
    @contextlib.contextmanager
    def with_grad(cls):
        old, cls._grad.on = cls.grad_enabled(), True
        try:
            yield
        finally:
            cls._grad.on = old

    @classmethod
    @contextlib.contextmanager
    def no_grad(cls):
        old, cls._grad.on = cls.grad_enabled(), False
        try:
            yield
        finally:
            cls._grad.on = old


@dataclass
class _Node:
    id: int
    op: str
    inputs: list
    backward_fn: Callable | None
    grad: torch.Tensor | None = None


class DynamicGraph:
    """Define-by-run graph: nodes get ids in creation order; ``backward`` walks ids in descending order."""

    def __init__(self):
        self.nodes: dict[int, _Node] = {}
        self.recording = True
        self._next = 0

    def add_node(self, op, inputs, backward_fn=None) -> int:
        nid = self._next
        self._next += 1
        if self.recording and DynamicContext.grad_enabled():
            self.nodes[nid] = _Node(nid, op, list(inputs), backward_fn)
        return nid

    def backward(self, node_id: int, grad: torch.Tensor):
        self.nodes[node_id].grad = grad
        for nid in sorted(self.nodes, reverse=True):
            n = self.nodes[nid]
            if n.grad is None or n.backward_fn is None:
                continue
            for iid, g in zip(n.inputs, n.backward_fn(n.grad)):
                if iid in self.nodes and g is not None:
                    m = self.nodes[iid]
                    m.grad = g if m.grad is None else m.grad + g

    def grad_of(self, node_id: int):
        return self.nodes[node_id].grad

    def clear(self):
        self.nodes.clear()
        self._next = 0


class DynamicTensor:
    """Tensor bound to a :class:`DynamicGraph`; supports add, mul, matmul, relu and backward."""

    def __init__(self, data, graph: DynamicGraph | None = None, _node=None):
        self.data = _unwrap(data) if not isinstance(data, torch.Tensor) else data
        self.graph = graph or DynamicGraph()
        self.node = self.graph.add_node("leaf", []) if _node is None else _node

    def _new(self, data, op, inputs, fn):
        return DynamicTensor(data, self.graph, self.graph.add_node(op, inputs, fn))

    def add(self, o):
        return self._new(self.data + o.data, "add", [self.node, o.node], lambda g: grad_fns.add_backward(g))

    def mul(self, o):
        a, b = self.data, o.data
        return self._new(a * b, "mul", [self.node, o.node], lambda g: grad_fns.mul_backward(g, a, b))

    def matmul(self, o):
        a, b = self.data, o.data
        return self._new(a @ b, "matmul", [self.node, o.node], lambda g: grad_fns.matmul_backward(g, a, b))

    def relu(self):
        x = self.data
        return self._new(torch.relu(x), "relu", [self.node], lambda g: (grad_fns.relu_backward(g, x),))

    def sum(self):
        x = self.data
        return self._new(x.sum(), "sum", [self.node], lambda g: (g * torch.ones_like(x),))

    __add__, __mul__, __matmul__ = add, mul, matmul

    def backward(self, grad=None):
        self.graph.backward(self.node, torch.ones_like(self.data) if grad is None else grad)

    @property
    def grad(self):
        g = self.graph.grad_of(self.node) if self.node in self.graph.nodes else None
        return Tensor(g) if g is not None else None
