"""Weight initialisers with the reference's names and bounds (ghostflow-nn/src/init.rs:7-89):
xavier_uniform bound sqrt(6/(fan_in+fan_out)), kaiming_uniform bound sqrt(6/fan_in). They fill a tensor
in place (and return it) or create one from a shape."""
from __future__ import annotations

import math

import torch


def _fans(shape):
    if len(shape) < 2:
        return shape[0], shape[0]
    rf = 1
    for s in shape[2:]:
        rf *= s
    return shape[1] * rf, shape[0] * rf


def _target(t_or_shape, device=None, dtype=torch.float32):
    if isinstance(t_or_shape, torch.Tensor):
        return t_or_shape
    return torch.empty(tuple(t_or_shape), device=device, dtype=dtype)


@torch.no_grad()
def xavier_uniform(t, gain: float = 1.0, generator=None):
    t = _target(t)
    fi, fo = _fans(t.shape)
    b = gain * math.sqrt(6.0 / (fi + fo))
    return t.uniform_(-b, b, generator=generator)


@torch.no_grad()
def xavier_normal(t, gain: float = 1.0, generator=None):
    t = _target(t)
    fi, fo = _fans(t.shape)
    return t.normal_(0.0, gain * math.sqrt(2.0 / (fi + fo)), generator=generator)


@torch.no_grad()
def kaiming_uniform(t, generator=None):
    t = _target(t)
    fi, _ = _fans(t.shape)
    b = math.sqrt(6.0 / fi)
    return t.uniform_(-b, b, generator=generator)


@torch.no_grad()
def kaiming_normal(t, generator=None):
    t = _target(t)
    fi, _ = _fans(t.shape)
    return t.normal_(0.0, math.sqrt(2.0 / fi), generator=generator)


@torch.no_grad()
def uniform(t, low: float = 0.0, high: float = 1.0, generator=None):
    return _target(t).uniform_(low, high, generator=generator)


@torch.no_grad()
def normal(t, mean: float = 0.0, std: float = 1.0, generator=None):
    return _target(t).normal_(mean, std, generator=generator)


@torch.no_grad()
def constant(t, value: float):
    return _target(t).fill_(value)


@torch.no_grad()
def zeros(t):
    return _target(t).zero_()


@torch.no_grad()
def ones(t):
    return _target(t).fill_(1.0)
