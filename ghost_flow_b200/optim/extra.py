"""RMSprop, AdaGrad and Adadelta.

The reference names these three beside SGD/Adam/AdamW in the optimizer list of its disabled deep-learning catalogue
(ghostflow-ml/src/lib.rs:133-134, ``deep/optimizers``); they share the :class:`Optimizer` interface of
ghostflow-optim/src/optimizer.rs:6-21 (``step, zero_grad, get_lr, set_lr``). The update of a whole parameter group is
issued as multi-tensor (``torch._foreach_*``) operations, so the number of launches does not grow with the number
of parameters; the formulas are the textbook ones (Tieleman & Hinton 2012; Duchi et al. 2011; Zeiler 2012).
"""
from __future__ import annotations

import torch

from .optimizers import Optimizer


def _active(group):
    ps = [p for p in group["params"] if p.grad is not None]
    return ps, [p.grad for p in ps]


class _StatefulOptimizer(Optimizer):
    def _buffers(self, ps, name: str, fill: float = 0.0):
        out = []
        for p in ps:
            st = self.state.setdefault(id(p), {})
            if name not in st:
                st[name] = torch.full_like(p, fill, dtype=torch.float32 if p.dtype != torch.float64 else p.dtype)
            out.append(st[name])
        return out

    @staticmethod
    def _decayed(ps, gs, wd: float):
        gs = [g.float() if g.dtype in (torch.bfloat16, torch.float16) else g for g in gs]
        if wd != 0.0:
            gs = torch._foreach_add(gs, [p.to(g.dtype) for p, g in zip(ps, gs)], alpha=wd)
        return gs

    @staticmethod
    def _apply(ps, updates, lr: float):
        """p -= lr * update, in the parameter's own dtype."""
        same = [u if u.dtype == p.dtype else u.to(p.dtype) for p, u in zip(ps, updates)]
        torch._foreach_add_(ps, same, alpha=-lr)


class RMSprop(_StatefulOptimizer):
    """``v = a v + (1-a) g^2`` (``centered``: minus the squared running mean of g); ``p -= lr g / (sqrt(v) + eps)``,
    optionally through a momentum buffer."""

    def __init__(self, params, lr: float = 0.01, alpha: float = 0.99, eps: float = 1e-8, weight_decay: float = 0.0,
                 momentum: float = 0.0, centered: bool = False):
        super().__init__(params, dict(lr=lr, alpha=alpha, eps=eps, weight_decay=weight_decay, momentum=momentum,
                                      centered=centered))

    @torch.no_grad()
    def step(self):
        self.step_count += 1
        for g in self.param_groups:
            ps, gs = _active(g)
            if not ps:
                continue
            gs = self._decayed(ps, gs, g["weight_decay"])
            sq = self._buffers(ps, "square_avg")
            torch._foreach_mul_(sq, g["alpha"])
            torch._foreach_addcmul_(sq, gs, gs, value=1 - g["alpha"])
            if g["centered"]:
                avg = self._buffers(ps, "grad_avg")
                torch._foreach_lerp_(avg, gs, 1 - g["alpha"])
                denom = torch._foreach_addcmul(sq, avg, avg, value=-1.0)
                torch._foreach_clamp_min_(denom, 0.0)
                torch._foreach_sqrt_(denom)
            else:
                denom = torch._foreach_sqrt(sq)
            torch._foreach_add_(denom, g["eps"])
            upd = torch._foreach_div(gs, denom)
            if g["momentum"] > 0:
                buf = self._buffers(ps, "momentum_buffer")
                torch._foreach_mul_(buf, g["momentum"])
                torch._foreach_add_(buf, upd)
                upd = buf
            self._apply(ps, upd, g["lr"])


class AdaGrad(_StatefulOptimizer):
    """``s += g^2``; ``p -= lr / (1 + (t-1) lr_decay) * g / (sqrt(s) + eps)``."""

    def __init__(self, params, lr: float = 0.01, lr_decay: float = 0.0, weight_decay: float = 0.0,
                 initial_accumulator_value: float = 0.0, eps: float = 1e-10):
        super().__init__(params, dict(lr=lr, lr_decay=lr_decay, weight_decay=weight_decay,
                                      initial_accumulator_value=initial_accumulator_value, eps=eps))

    @torch.no_grad()
    def step(self):
        self.step_count += 1
        for g in self.param_groups:
            ps, gs = _active(g)
            if not ps:
                continue
            gs = self._decayed(ps, gs, g["weight_decay"])
            acc = self._buffers(ps, "sum", g["initial_accumulator_value"])
            torch._foreach_addcmul_(acc, gs, gs, value=1.0)
            denom = torch._foreach_sqrt(acc)
            torch._foreach_add_(denom, g["eps"])
            clr = g["lr"] / (1.0 + (self.step_count - 1) * g["lr_decay"])
            self._apply(ps, torch._foreach_div(gs, denom), clr)


Adagrad = AdaGrad


class Adadelta(_StatefulOptimizer):
    """``v = rho v + (1-rho) g^2``; ``d = sqrt(u + eps) / sqrt(v + eps) * g``; ``u = rho u + (1-rho) d^2``;
    ``p -= lr d``."""

    def __init__(self, params, lr: float = 1.0, rho: float = 0.9, eps: float = 1e-6, weight_decay: float = 0.0):
        super().__init__(params, dict(lr=lr, rho=rho, eps=eps, weight_decay=weight_decay))

    @torch.no_grad()
    def step(self):
        self.step_count += 1
        for g in self.param_groups:
            ps, gs = _active(g)
            if not ps:
                continue
            gs = self._decayed(ps, gs, g["weight_decay"])
            sq = self._buffers(ps, "square_avg")
            acc = self._buffers(ps, "acc_delta")
            rho, eps = g["rho"], g["eps"]
            torch._foreach_mul_(sq, rho)
            torch._foreach_addcmul_(sq, gs, gs, value=1 - rho)
            std = torch._foreach_add(sq, eps)
            torch._foreach_sqrt_(std)
            delta = torch._foreach_add(acc, eps)
            torch._foreach_sqrt_(delta)
            torch._foreach_div_(delta, std)
            torch._foreach_mul_(delta, gs)
            torch._foreach_mul_(acc, rho)
            torch._foreach_addcmul_(acc, delta, delta, value=1 - rho)
            self._apply(ps, delta, g["lr"])
