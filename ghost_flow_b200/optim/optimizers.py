"""SGD, Adam and AdamW with the reference's semantics (ghostflow-optim/src/sgd.rs:17-93, adam.rs:19-197,
optimizer.rs:6-43), operating on the model's own parameters (the reference updates clones, so a model never
sees its update: adam.rs:194, ghostflow-nn/src/linear.rs:71-77).

CUDA parameters are grouped into flat fp32 buffers so that one fused kernel launch updates every
parameter of a group (``gf_adam_flat`` / ``gf_sgd_flat``); bf16 parameters keep an fp32 master copy in
that buffer. CPU parameters use the plain per-tensor formulas.
"""
from __future__ import annotations

import math
from typing import Iterable

import torch

from ..ops import _lib
from ..tensor import Tensor


def _params(params):
    out = []
    for p in params:
        if isinstance(p, dict):
            out.append({**p, "params": [q.data if isinstance(q, Tensor) else q for q in p["params"]]})
        else:
            out.append(p.data if isinstance(p, Tensor) else p)
    return out


class ParamGroup(dict):
    """``{params, lr, weight_decay, ...}`` (ghostflow-optim/src/optimizer.rs:24-43)."""


class Optimizer:
    """Base class: ``step, zero_grad, get_lr, set_lr, parameters`` (ghostflow-optim/src/optimizer.rs:6-21)."""

    def __init__(self, params, defaults: dict):
        params = _params(list(params))
        if params and isinstance(params[0], dict):
            self.param_groups = [ParamGroup({**defaults, **g}) for g in params]
        else:
            self.param_groups = [ParamGroup({**defaults, "params": params})]
        self.state: dict = {}
        self._flat: dict = {}
        self.step_count = 0

    # -- reference API
    @classmethod
    def new(cls, *args, **kwargs):
        """``SGD.new(params, 0.01)``: the reference's constructor spelling."""
        return cls(*args, **kwargs)

    def get_lr(self) -> float:
        return self.param_groups[0]["lr"]

    def set_lr(self, lr: float) -> None:
        for g in self.param_groups:
            g["lr"] = lr

    def parameters(self):
        return [p for g in self.param_groups for p in g["params"]]

    def zero_grad(self, set_to_none: bool = True) -> None:
        for p in self.parameters():
            if p.grad is not None:
                if set_to_none:
                    p.grad = None
                else:
                    p.grad.zero_()

    # -- flat CUDA buffers
    def _flat_group(self, gi: int, n_state: int):
        """Lazily builds [master, state...] fp32 flat buffers for the CUDA params of group ``gi``."""
        f = self._flat.get(gi)
        if f is not None:
            return f
        ps = [p for p in self.param_groups[gi]["params"] if p.is_cuda and p.requires_grad]
        if not ps:
            self._flat[gi] = None
            return None
        offs, n = [], 0
        for p in ps:
            offs.append(n)
            n += (p.numel() + 3) // 4 * 4
        dev = ps[0].device
        master = torch.zeros(n, dtype=torch.float32, device=dev)
        for p, o in zip(ps, offs):
            master[o:o + p.numel()] = p.detach().reshape(-1).float()
            if p.dtype == torch.float32 and p.is_contiguous():
                # fp32 parameters need no second copy: they become views of the flat buffer, so whatever else writes
                # them (load_state_dict, clamping, an EMA swap) writes the optimizer's copy too
                p.data = master[o:o + p.numel()].view(p.shape)
        f = {"params": ps, "offs": offs, "n": n, "master": master,
             "state": [torch.zeros(n, dtype=torch.float32, device=dev) for _ in range(n_state)],
             "grad": torch.zeros(n, dtype=torch.float32, device=dev),
             "is_view": [p.dtype == torch.float32 and p.data_ptr() == master[o:o + 1].data_ptr()
                         for p, o in zip(ps, offs)],
             "versions": [p._version for p in ps]}
        self._flat[gi] = f
        return f

    @staticmethod
    def _sync_master(f):
        """Low-precision parameters keep an fp32 master copy in the flat buffer. If such a parameter was written
        from outside since the last step (``load_state_dict``, ``p.copy_``, ``p.clamp_`` under ``no_grad``: anything
        that bumps its version counter), the master copy is refreshed from it; otherwise the next step would put
        the old value back. Writes through ``p.data`` leave no trace and are not seen."""
        for i, (p, o) in enumerate(zip(f["params"], f["offs"])):
            if f["is_view"][i]:
                continue
            if p._version != f["versions"][i]:
                f["master"][o:o + p.numel()] = p.detach().reshape(-1).float()
                f["versions"][i] = p._version

    @staticmethod
    def _gather_grads(f):
        """Copies the gradients into the flat buffer and returns it with the element ranges ``[(lo, hi), ...]``
        that have one. A parameter without a gradient in this step is left out of the update altogether (no
        weight decay, no decay of its moments), like the per-tensor path and the reference's loop do."""
        g = f["grad"]
        runs, lo, hi = [], None, None
        for p, o in zip(f["params"], f["offs"]):
            if p.grad is None:
                if lo is not None:
                    runs.append((lo, hi))
                    lo = None
                continue
            g[o:o + p.numel()].copy_(p.grad.reshape(-1))
            end = o + (p.numel() + 3) // 4 * 4
            if lo is None:
                lo = o
            hi = end
        if lo is not None:
            runs.append((lo, hi))
        return g, runs

    @staticmethod
    def _scatter_params(f):
        m = f["master"]
        for i, (p, o) in enumerate(zip(f["params"], f["offs"])):
            if not f["is_view"][i]:
                p.data.copy_(m[o:o + p.numel()].view_as(p))

    def state_dict(self):
        return {"step": self.step_count, "param_groups": [{k: v for k, v in g.items() if k != "params"}
                                                            for g in self.param_groups],
                "state": {k: {kk: vv.clone() if torch.is_tensor(vv) else vv for kk, vv in v.items()}
                          for k, v in self.state.items()},
                "flat": {gi: {"master": f["master"].clone(), "state": [s.clone() for s in f["state"]]}
                         for gi, f in self._flat.items() if f is not None}}

    def load_state_dict(self, sd):
        self.step_count = sd["step"]
        for g, saved in zip(self.param_groups, sd["param_groups"]):
            g.update(saved)
        self.state = {k: dict(v) for k, v in sd.get("state", {}).items()}
        for gi, saved in sd.get("flat", {}).items():
            f = self._flat_group(int(gi), len(saved["state"]))
            f["master"].copy_(saved["master"])
            for a, b in zip(f["state"], saved["state"]):
                a.copy_(b)


class SGD(Optimizer):
    """``g += wd*p; v = mu*v + (1-damp)*g; nesterov: g += mu*v else g = v; p -= lr*g``."""

    def __init__(self, params, lr: float = 0.01, momentum: float = 0.0, weight_decay: float = 0.0,
                 dampening: float = 0.0, nesterov: bool = False):
        super().__init__(params, dict(lr=lr, momentum=momentum, weight_decay=weight_decay, dampening=dampening,
                                      nesterov=nesterov))

    # builder-style setters of the reference
    def momentum(self, v): return self._set("momentum", v)
    def weight_decay(self, v): return self._set("weight_decay", v)
    def dampening(self, v): return self._set("dampening", v)
    def nesterov(self, v=True): return self._set("nesterov", v)

    def _set(self, k, v):
        for g in self.param_groups:
            g[k] = v
        return self

    @torch.no_grad()
    def step(self):
        self.step_count += 1
        for gi, g in enumerate(self.param_groups):
            f = self._flat_group(gi, 1)
            if f is not None:
                from ..ops.optim_kernels import sgd_flat

                self._sync_master(f)
                grads, runs = self._gather_grads(f)
                with torch.cuda.device(f["master"].device):
                    for lo, hi in runs:
                        sgd_flat(f["master"][lo:hi], f["state"][0][lo:hi], grads[lo:hi], None, lr=g["lr"],
                                 momentum=g["momentum"], dampening=g["dampening"], weight_decay=g["weight_decay"],
                                 nesterov=g["nesterov"], first_step=(self.step_count == 1))
                self._scatter_params(f)
            for p in g["params"]:
                if p.is_cuda or p.grad is None:
                    continue
                d = p.grad
                if g["weight_decay"] != 0:
                    d = d.add(p, alpha=g["weight_decay"])
                if g["momentum"] != 0:
                    st = self.state.setdefault(id(p), {})
                    buf = st.get("momentum_buffer")
                    if buf is None:
                        buf = st["momentum_buffer"] = d.clone()
                    else:
                        buf.mul_(g["momentum"]).add_(d, alpha=1 - g["dampening"])
                    d = d.add(buf, alpha=g["momentum"]) if g["nesterov"] else buf
                p.add_(d, alpha=-g["lr"])


class Adam(Optimizer):
    """Adam with bias correction; ``weight_decay`` is L2-coupled (added to the gradient)."""
    decoupled = False

    def __init__(self, params, lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 0.0):
        super().__init__(params, dict(lr=lr, betas=tuple(betas), eps=eps, weight_decay=weight_decay))

    def betas(self, b1, b2):
        for g in self.param_groups:
            g["betas"] = (b1, b2)
        return self

    def eps(self, e):
        for g in self.param_groups:
            g["eps"] = e
        return self

    def weight_decay(self, wd):
        for g in self.param_groups:
            g["weight_decay"] = wd
        return self

    @torch.no_grad()
    def step(self):
        self.step_count += 1
        t = self.step_count
        for gi, g in enumerate(self.param_groups):
            b1, b2 = g["betas"]
            f = self._flat_group(gi, 2)
            if f is not None:
                from ..ops.optim_kernels import adam_flat

                self._sync_master(f)
                grads, runs = self._gather_grads(f)
                with torch.cuda.device(f["master"].device):
                    for lo, hi in runs:
                        adam_flat(f["master"][lo:hi], f["state"][0][lo:hi], f["state"][1][lo:hi], grads[lo:hi], None,
                                  lr=g["lr"], beta1=b1, beta2=b2, eps=g["eps"], weight_decay=g["weight_decay"], step=t,
                                  decoupled=self.decoupled)
                self._scatter_params(f)
            for p in g["params"]:
                if p.is_cuda or p.grad is None:
                    continue
                st = self.state.setdefault(id(p), {})
                if "exp_avg" not in st:
                    st["exp_avg"] = torch.zeros_like(p, dtype=torch.float32)
                    st["exp_avg_sq"] = torch.zeros_like(p, dtype=torch.float32)
                grad = p.grad.float()
                if not self.decoupled and g["weight_decay"] != 0:
                    grad = grad.add(p.float(), alpha=g["weight_decay"])
                m, v = st["exp_avg"], st["exp_avg_sq"]
                m.mul_(b1).add_(grad, alpha=1 - b1)
                v.mul_(b2).addcmul_(grad, grad, value=1 - b2)
                mh = m / (1 - b1 ** t)
                vh = v / (1 - b2 ** t)
                if self.decoupled and g["weight_decay"] != 0:
                    p.mul_(1 - g["lr"] * g["weight_decay"])
                p.add_((-g["lr"] * mh / (vh.sqrt() + g["eps"])).to(p.dtype))


class AdamW(Adam):
    """``p*(1 - lr*wd) - lr * mhat / (sqrt(vhat) + eps)``; default weight decay 0.01 (adam.rs:129-197)."""
    decoupled = True

    def __init__(self, params, lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 0.01):
        super().__init__(params, lr, betas, eps, weight_decay)


def clip_grad_norm_(params, max_norm: float, norm_type: float = 2.0) -> torch.Tensor:
    """Scales gradients so that their global norm is at most ``max_norm``; returns the norm before clipping.
    (The reference advertises clipping, README.md:93-97, without implementing it.)"""
    ps = [p.data if isinstance(p, Tensor) else p for p in params]
    grads = [p.grad for p in ps if p.grad is not None]
    if not grads:
        return torch.tensor(0.0)
    if norm_type == math.inf:
        total = max(g.abs().max() for g in grads)
    else:
        total = torch.norm(torch.stack([torch.norm(g.float(), norm_type) for g in grads]), norm_type)
    coef = (max_norm / (total + 1e-6)).clamp(max=1.0)
    for g in grads:
        g.mul_(coef.to(g.dtype))
    return total
