"""Shared plumbing of the classical-ML package: array conversion, fluent builder setters, estimator mixins.

Convention of the reference (ghostflow-ml, every file): ``X`` is ``[n_samples, n_features]`` float32, ``y`` is
``[n_samples]`` float32 with class ids stored as floats; builder methods return the estimator; ``fit`` / ``predict``
/ ``predict_proba`` / ``transform``. Inputs here may be :class:`ghost_flow_b200.Tensor`, torch tensors, numpy
arrays or nested lists; outputs are :class:`ghost_flow_b200.Tensor` (float32). The algorithms run in float64 numpy
on the host: this package is deliberately off the GPU hot path.
"""
from __future__ import annotations

import numpy as np
import torch

from ..tensor import Tensor


def to_np(x, dtype=np.float64) -> np.ndarray:
    if isinstance(x, Tensor):
        x = x.data
    if isinstance(x, torch.Tensor):
        x = x.detach().cpu().float().numpy() if x.is_floating_point() else x.detach().cpu().numpy()
    a = np.asarray(x)
    return a.astype(dtype) if dtype is not None else a


def out(a) -> Tensor:
    return Tensor(torch.from_numpy(np.ascontiguousarray(np.asarray(a, dtype=np.float32))))


def rng_of(seed):
    return np.random.default_rng(seed)


class Estimator:
    """Fluent setters: ``Model().max_depth(4).learning_rate(0.1)`` sets same-named attributes (stored with a leading
    underscore when a method of that name exists). ``set(name=value, ...)`` does the same for several at once."""

    _params: tuple = ()

    def __init_subclass__(cls, **kw):
        super().__init_subclass__(**kw)
        for name in cls._params:
            if name not in cls.__dict__:
                setattr(cls, name, _make_setter(name))

    def set(self, **kw):
        for k, v in kw.items():
            setattr(self, "_" + k, _plain(v))
        return self

    def get_params(self) -> dict:
        return {k: getattr(self, "_" + k, None) for k in self._all_params()}

    @classmethod
    def _all_params(cls):
        seen = []
        for c in reversed(cls.__mro__):
            for p in getattr(c, "_params", ()):
                if p not in seen:
                    seen.append(p)
        return seen

    def clone(self):
        import copy
        return copy.deepcopy(self)


def _plain(value):
    """Option enums (``ml.options``) are stored as the strings the algorithms compare against."""
    import enum

    return value.value if isinstance(value, enum.Enum) else value


def _make_setter(name):
    def setter(self, value):
        setattr(self, "_" + name, _plain(value))
        return self
    setter.__name__ = name
    return setter


class ClassifierMixin:
    def score(self, X, y) -> float:
        return float((to_np(self.predict(X)) == to_np(y)).mean())


class RegressorMixin:
    def score(self, X, y) -> float:
        y = to_np(y)
        p = to_np(self.predict(X))
        ss_res = ((y - p) ** 2).sum()
        ss_tot = ((y - y.mean()) ** 2).sum()
        return float(1.0 - ss_res / ss_tot) if ss_tot > 0 else 0.0


class TransformerMixin:
    def fit_transform(self, X, y=None):
        return self.fit(X, y).transform(X) if y is not None else self.fit(X).transform(X)


def encode_classes(y):
    """(sorted class values, integer codes)."""
    classes, codes = np.unique(to_np(y), return_inverse=True)
    return classes, codes


def softmax(z):
    z = z - z.max(axis=1, keepdims=True)
    e = np.exp(z)
    return e / e.sum(axis=1, keepdims=True)


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-np.clip(z, -60, 60)))


def pairwise_sq_dists(A, B):
    d = (A * A).sum(1)[:, None] + (B * B).sum(1)[None, :] - 2.0 * A @ B.T
    return np.maximum(d, 0.0)
