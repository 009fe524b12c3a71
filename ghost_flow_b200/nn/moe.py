"""Mixture of experts (ghostflow-nn/src/mixture_of_experts.rs:14-385): ``RoutingStrategy``, ``MoEConfig`` presets
(default 8 experts / top-2 / capacity 1.25 / aux weight 0.01, ``switch_transformer``, ``gshard``, ``expert_choice``),
``Expert``, ``Router.route / select_top_k``, ``MixtureOfExperts.forward / get_aux_loss / get_expert_usage /
load_balance_factor / get_stats``.

Math kept from the reference: softmax over all experts, top-k, output = sum_k w_k * expert_k(x) / sum_k w_k
(:152-177, :236-261). The per-token loop becomes a sort by expert + one grouped pass per expert. Two auxiliary
losses are exposed: the standard load-balancing loss ``E * sum_e f_e * P_e`` used for training, and the reference's
coefficient-of-variation statistic (:313-322) in ``MoEStats``. Experts are GELU two-matrix FFNs like the
reference's, or SwiGLU (``expert_type="swiglu"``) for Mixtral-style models. ``ExpertChoice`` routing and the
capacity factor, which the reference declares and never reads, are implemented.
"""
from __future__ import annotations

import enum
from dataclasses import dataclass

import torch
import torch.nn.functional as F

from .. import ops
from .layers import Linear
from .module import Module, ModuleList


class RoutingStrategy(enum.Enum):
    TopK = "top_k"
    Switch = "switch"
    ExpertChoice = "expert_choice"


@dataclass
class MoEConfig:
    num_experts: int = 8
    top_k: int = 2
    d_model: int = 512
    d_ff: int = 2048
    capacity_factor: float = 1.25
    aux_loss_weight: float = 0.01
    routing: RoutingStrategy = RoutingStrategy.TopK
    expert_parallel: bool = False
    expert_dropout: float = 0.0
    expert_type: str = "gelu"       # "gelu" (reference) or "swiglu" (Mixtral)
    drop_tokens: bool = False       # False = dropless (capacity factor only reported)

    @classmethod
    def default(cls): return cls()
    @classmethod
    def switch_transformer(cls, num_experts=128): return cls(num_experts, 1, routing=RoutingStrategy.Switch)
    @classmethod
    def gshard(cls, num_experts=64): return cls(num_experts, 2, capacity_factor=2.0)
    @classmethod
    def expert_choice(cls, num_experts=8): return cls(num_experts, 2, routing=RoutingStrategy.ExpertChoice)


@dataclass
class MoEStats:
    expert_usage: list
    load_balance_factor: float
    aux_loss: float
    cv_aux_loss: float
    dropped_tokens: int = 0


class Expert(Module):
    def __init__(self, d_model: int, d_ff: int, expert_type: str = "gelu", device=None, dtype=None):
        super().__init__()
        self.expert_type = expert_type
        if expert_type == "swiglu":
            self.w1 = Linear(d_model, 2 * d_ff, False, device, dtype)   # gate | up
        else:
            self.w1 = Linear(d_model, d_ff, False, device, dtype)
        self.w2 = Linear(d_ff, d_model, False, device, dtype)

    def forward(self, x):
        h = self.w1(x)
        h = ops.swiglu(h) if self.expert_type == "swiglu" else ops.gelu(h)
        return self.w2(h)


class Router(Module):
    def __init__(self, d_model: int, num_experts: int, device=None, dtype=None):
        super().__init__()
        self.gate = Linear(d_model, num_experts, False, device, dtype)

    def route(self, x):
        """Router probabilities ``[tokens, experts]`` (fp32 softmax over all experts)."""
        return torch.softmax(self.gate(x).float(), dim=-1)

    @staticmethod
    def select_top_k(probs, k: int):
        w, idx = torch.topk(probs, k, dim=-1)
        return w, idx

    forward = route


class MixtureOfExperts(Module):
    def __init__(self, config: MoEConfig | None = None, device=None, dtype=None):
        super().__init__()
        self.config = c = config or MoEConfig()
        self.router = Router(c.d_model, c.num_experts, device, dtype)
        self.experts = ModuleList([Expert(c.d_model, c.d_ff, c.expert_type, device, dtype)
                                   for _ in range(c.num_experts)])
        self._aux = None
        self._cv = None
        self._usage = torch.zeros(c.num_experts)
        self._dropped = 0

    def forward(self, x):
        c = self.config
        shape = x.shape
        t = x.reshape(-1, shape[-1])
        T, E = t.shape[0], c.num_experts
        probs = self.router.route(t)
        if c.routing == RoutingStrategy.ExpertChoice:
            out = self._expert_choice(t, probs)
        else:
            k = 1 if c.routing == RoutingStrategy.Switch else c.top_k
            w, idx = Router.select_top_k(probs, k)
            w = w / w.sum(-1, keepdim=True)
            flat_e = idx.reshape(-1)
            order = torch.argsort(flat_e, stable=True)
            tok = order // k
            counts = torch.bincount(flat_e, minlength=E)
            self._dropped = 0
            keep = None
            if c.drop_tokens:
                cap = int(c.capacity_factor * T * k / E)
                pos = torch.arange(order.numel(), device=t.device) - torch.repeat_interleave(
                    torch.cumsum(counts, 0) - counts, counts)
                keep = pos < cap
                self._dropped = int((~keep).sum())
            xs = t.index_select(0, tok)
            ys = torch.empty_like(xs)
            start = 0
            counts_l = counts.tolist()
            for e in range(E):
                n = counts_l[e]
                if n:
                    ys[start:start + n] = self.experts[e](xs[start:start + n])
                start += n
            wsel = w.reshape(-1)[order].to(ys.dtype).unsqueeze(-1)
            if keep is not None:
                wsel = wsel * keep.unsqueeze(-1)
            out = torch.zeros_like(t).index_add_(0, tok, ys * wsel)
            # standard load-balancing loss: E * sum_e (fraction of assignments to e) * (mean router prob of e)
            f = counts.float() / max(1, flat_e.numel())
            self._aux = E * torch.sum(f * probs.mean(0))
            self._usage = counts.detach().float().cpu()
        mean_p = probs.mean(0)
        self._cv = (mean_p.std(unbiased=False) / mean_p.mean().clamp(min=1e-12)) * c.aux_loss_weight
        if c.routing == RoutingStrategy.ExpertChoice:
            self._aux = torch.zeros((), device=t.device)
        return out.reshape(shape)

    def _expert_choice(self, t, probs):
        """Each expert picks its top ``capacity`` tokens (perfect balance by construction)."""
        c = self.config
        T, E = probs.shape
        cap = max(1, int(c.capacity_factor * T * c.top_k / E))
        cap = min(cap, T)
        w, tok = torch.topk(probs.t(), cap, dim=-1)     # [E, cap]
        out = torch.zeros_like(t)
        for e in range(E):
            ye = self.experts[e](t.index_select(0, tok[e]))
            out.index_add_(0, tok[e], ye * w[e].to(ye.dtype).unsqueeze(-1))
        self._usage = torch.full((E,), float(cap))
        return out

    def get_aux_loss(self):
        """Load-balancing loss times ``aux_loss_weight`` (add it to the training loss)."""
        if self._aux is None:
            return torch.zeros(())
        return self._aux * self.config.aux_loss_weight

    def get_expert_usage(self):
        return self._usage.tolist()

    def load_balance_factor(self) -> float:
        """min / max expert load of the last forward (1.0 = perfectly balanced)."""
        u = self._usage
        return float(u.min() / u.max().clamp(min=1.0)) if u.numel() else 1.0

    def get_stats(self) -> MoEStats:
        return MoEStats(self.get_expert_usage(), self.load_balance_factor(), float(self.get_aux_loss().detach()),
                        float(self._cv) if self._cv is not None else 0.0, self._dropped)
