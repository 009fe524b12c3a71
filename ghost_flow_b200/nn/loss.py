"""Loss functions with the reference's names (ghostflow-nn/src/loss.rs:6-293): functional forms plus thin
module classes. ``cross_entropy`` takes ``[N, C]`` (or ``[..., C]``) logits and class ids (integer or
float tensors, the reference stores targets as f32); on bf16 CUDA logits it runs the fused softmax-xent
kernel that produces the loss and the logits gradient in one pass over HBM."""
from __future__ import annotations

import torch
import torch.nn.functional as F

from .. import ops
from ..tensor import Tensor
from .module import Module


def _u(x):
    return x.data if isinstance(x, Tensor) else x


def _w(fn):
    def wrapped(*args, **kw):
        wrapped_in = any(isinstance(a, Tensor) for a in args)
        out = fn(*[_u(a) for a in args], **kw)
        return Tensor(out) if wrapped_in else out

    wrapped.__name__ = fn.__name__
    wrapped.__doc__ = fn.__doc__
    return wrapped


@_w
def mse_loss(pred, target):
    return F.mse_loss(pred, target)


@_w
def l1_loss(pred, target):
    return F.l1_loss(pred, target)


@_w
def smooth_l1_loss(pred, target, beta: float = 1.0):
    return F.smooth_l1_loss(pred, target, beta=beta)


@_w
def huber_loss(pred, target, delta: float = 1.0):
    return F.huber_loss(pred, target, delta=delta)


@_w
def binary_cross_entropy(pred, target, eps: float = 1e-7):
    p = pred.clamp(eps, 1 - eps)
    return -(target * p.log() + (1 - target) * (1 - p).log()).mean()


@_w
def binary_cross_entropy_with_logits(logits, target):
    return F.binary_cross_entropy_with_logits(logits, target)


@_w
def cross_entropy(logits, target, ignore_index=None):
    """Mean of ``-log_softmax(logits)[target]`` over rows."""
    tgt = target.long() if target.is_floating_point() else target
    return ops.cross_entropy(logits, tgt, ignore_index=ignore_index)


@_w
def nll_loss(log_probs, target):
    tgt = target.long() if target.is_floating_point() else target
    return F.nll_loss(log_probs, tgt)


@_w
def cosine_embedding_loss(x1, x2, target, margin: float = 0.0):
    return F.cosine_embedding_loss(x1, x2, target, margin=margin)


@_w
def triplet_margin_loss(anchor, positive, negative, margin: float = 1.0):
    return F.triplet_margin_loss(anchor, positive, negative, margin=margin)


@_w
def focal_loss(logits, target, alpha: float = 0.25, gamma: float = 2.0):
    tgt = target.long() if target.is_floating_point() else target
    logp = torch.log_softmax(logits.float(), -1).gather(-1, tgt.unsqueeze(-1)).squeeze(-1)
    p = logp.exp()
    return (-alpha * (1 - p) ** gamma * logp).mean()


@_w
def contrastive_loss(x1, x2, label, margin: float = 1.0):
    d = F.pairwise_distance(x1, x2)
    return (label * d.pow(2) + (1 - label) * (margin - d).clamp(min=0).pow(2)).mean()


@_w
def kl_div_loss(log_q, p):
    return F.kl_div(log_q, p, reduction="batchmean")


class _LossModule(Module):
    fn = None

    def __init__(self, **kw):
        super().__init__()
        self.kw = kw

    def forward(self, *args):
        return type(self).fn(*args, **self.kw)


class MSELoss(_LossModule):
    fn = staticmethod(mse_loss)


class L1Loss(_LossModule):
    fn = staticmethod(l1_loss)


class SmoothL1Loss(_LossModule):
    fn = staticmethod(smooth_l1_loss)


class HuberLoss(_LossModule):
    fn = staticmethod(huber_loss)


class BCELoss(_LossModule):
    fn = staticmethod(binary_cross_entropy)


class BCEWithLogitsLoss(_LossModule):
    fn = staticmethod(binary_cross_entropy_with_logits)


class CrossEntropyLoss(_LossModule):
    fn = staticmethod(cross_entropy)


class NLLLoss(_LossModule):
    fn = staticmethod(nll_loss)


class FocalLoss(_LossModule):
    fn = staticmethod(focal_loss)
