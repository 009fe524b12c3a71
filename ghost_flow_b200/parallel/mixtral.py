"""Mixtral-style mixture-of-experts decoder, trained with expert parallelism = world size.

The dense part of every layer (attention and the two norms) is a ZeRO-3 unit exactly as in
:class:`~ghost_flow_b200.parallel.zero3.Zero3LlamaEngine`: flat, sharded over the ranks, gathered for the layer,
gradients reduce-scattered into the fused AdamW. The MLP of a layer is ``num_local_experts`` SwiGLU experts owned
``experts / world`` per rank (:class:`~ghost_flow_b200.parallel.ep.ExpertParallelMoE`: router, dispatch and combine
over peer memory, grouped tcgen05 GEMMs); their weights, fp32 master copies and Adam moments never leave their
owner, so they need no collective at all: every rank already holds the full gradient of its experts, summed over
the tokens of all ranks that were routed there. The router weight is replicated; its gradient is all-reduced (a
``[experts, d]`` tensor). The loss is the next-token cross-entropy plus ``router_aux_loss_coef`` times the Switch
load-balancing loss ``E * sum_e f_e * P_e`` of every layer.

The reference's mixture of experts is a per-token CPU loop whose ``expert_parallel`` flag is never read
(ghostflow-nn/src/mixture_of_experts.rs:41,53,212-274) and whose auxiliary loss is a coefficient-of-variation
term (:289-323); there is no Mixtral preset (``MixtralConfig`` is ours, built on ``LLaMAConfig``).
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..models.configs import MixtralConfig
from ..ops import raw as K
from .ep import ExpertParallelMoE
from .zero3 import Comm, OptimConfig, Zero3LlamaEngine


class _ExpertState:
    """One layer's local experts and router: bf16 weights, fp32 master copies, Adam moments. The gradient buffers
    are the engine's: a layer's experts are updated as soon as its backward pass is over, so one set serves all."""

    def __init__(self, moe: ExpertParallelMoE, seed: int, std: float, init_device: str = "cpu"):
        dev = moe.device
        E, el, d, f = moe.E, moe.el, moe.d, moe.f
        lo = moe.rank * el
        # One generator per expert, seeded by (layer seed, expert): a rank draws its own experts only, and an expert's
        # weights do not depend on the world size. Drawn on the host by default (the same numbers on every device
        # type, which the tests against the CPU engine rely on); ``init_device="device"`` draws on the GPU, which a
        # 47 B-parameter model needs to start in seconds rather than minutes.
        gdev = dev if (init_device == "device" and dev.type == "cuda") else torch.device("cpu")

        def draw(sub_seed, *shape):
            g = torch.Generator(device=gdev).manual_seed(seed * 4099 + sub_seed)
            return (torch.randn(*shape, generator=g, device=gdev) * std).to(dev)

        gate = draw(0, E, d)
        w13 = torch.stack([draw(1 + 2 * e, 2 * f, d) for e in range(lo, lo + el)])
        w2 = torch.stack([draw(2 + 2 * e, d, f) for e in range(lo, lo + el)])
        lp = torch.bfloat16 if dev.type == "cuda" else torch.float32
        self.gate_pad = torch.zeros_like(moe.gate_pad, dtype=lp)
        self.master = {"gate": gate, "w13": w13, "w2": w2}
        self.gate_pad[:E] = self.master["gate"].to(self.gate_pad.dtype)
        self.w13 = self.master["w13"].to(lp) if lp != torch.float32 else self.master["w13"].clone()
        self.w2 = self.master["w2"].to(lp) if lp != torch.float32 else self.master["w2"].clone()
        self.m = {k: torch.zeros_like(v) for k, v in self.master.items()}
        self.v = {k: torch.zeros_like(v) for k, v in self.master.items()}

    def low_precision(self):
        return {"gate": self.gate_pad[:self.master["gate"].shape[0]], "w13": self.w13, "w2": self.w2}


class MixtralEngine(Zero3LlamaEngine):
    """ZeRO-3 over the attention / norm parameters, expert parallelism (one group of experts per rank) for the MLPs.

    ``tokens_per_rank`` (= micro-batch x sequence length) is fixed at construction: the dispatch buffers are sized
    for it. ``capacity_factor`` bounds the rows a rank accepts per layer (default 2.0; ``world`` is the drop-free
    worst case); an overflow is reported through the kernel status word.
    """

    def __init__(self, cfg: MixtralConfig, device, tokens_per_rank: int, optim: OptimConfig | None = None, group=None,
                 seed: int = 0, dtype=torch.bfloat16, comm: Comm | None = None, capacity_factor: float | None = None,
                 persist_gathered: bool | None = None, expert_init: str = "cpu"):
        super().__init__(cfg, device, optim=optim, group=group, seed=seed, dtype=dtype, comm=comm,
                         persist_gathered=persist_gathered)
        if self.opt.max_grad_norm is not None:
            raise NotImplementedError("gradient clipping is not wired into the expert optimizer yet")
        if self.recompute:
            raise NotImplementedError("activation recompute would dispatch every layer's tokens twice")
        E, k = cfg.num_local_experts, cfg.num_experts_per_tok
        cf = capacity_factor if capacity_factor is not None else (cfg.capacity_factor or 2.0)
        self.moe = ExpertParallelMoE(cfg.hidden_size, cfg.intermediate_size, E, k, tokens_per_rank, self.device,
                                     group=self.comm.group, capacity_factor=min(float(cf), float(self.world)) if self.world > 1 else 1.0,
                                     seed=seed, init_weights=False)
        self.moe.keep_slot_outputs = True
        self.moe.accumulate_grads = False      # one backward pass per step: gradients are written, not added
        # the loss is a mean over the ranks, and so is its auxiliary part: every rank adds coef / world of its own
        self.moe.aux_coef = float(cfg.router_aux_loss_coef) / self.world
        self.tokens_per_rank = tokens_per_rank
        self.experts = [_ExpertState(self.moe, seed * 7919 + 31 * i + 1, cfg.initializer_range, expert_init)
                        for i in range(cfg.num_hidden_layers)]
        e0 = self.experts[0]
        self.gate_grad_pad = torch.zeros_like(e0.gate_pad)
        self.g13, self.g2 = torch.zeros_like(e0.w13), torch.zeros_like(e0.w2)
        self.aux_losses: list = []

    def _layer_specs(self):
        c = self.cfg
        d, hd = c.hidden_size, c.head_dim
        return [("attn_norm", (d,)), ("wqkv", (self.qkv_out, d)), ("wo", (d, c.num_attention_heads * hd)),
                ("ffn_norm", (d,))]

    # ------------------------------------------------------------------ layer math
    def _use(self, i):
        e = self.experts[i]
        self.moe.set_weights(e.gate_pad, e.w13, e.w2, self.gate_grad_pad, self.g13, self.g2)
        return e

    def _layer_fwd(self, w, x, B, S, layer_index: int = 0):
        c = self.cfg
        x2, sa = self._attn_fwd(w, x, B, S)
        h2, rstd2, _ = K.rmsnorm_fwd(x2, w["ffn_norm"], c.rms_norm_eps)
        self._use(layer_index)
        out, ctx = self.moe.forward(h2.contiguous(), residual=x2)
        self.aux_losses.append(self.moe.aux_loss(ctx) if self.device.type == "cuda" else ctx[2].detach())
        return out.to(x.dtype), (sa, x2, rstd2, ctx)

    def _layer_bwd(self, w, g, saved, dout, B, S, layer_index: int = 0):
        sa, x2, rstd2, ctx = saved
        self._use(layer_index)
        dh2 = self.moe.backward(ctx, dout.contiguous())
        dx2, _ = K.rmsnorm_bwd(x2, w["ffn_norm"], dh2.to(x2.dtype), rstd2, dres=dout, dw_out=g["ffn_norm"])
        self._update_experts(layer_index)
        return self._attn_bwd(w, g, sa, dx2, B, S)

    def _update_experts(self, i):
        """AdamW on this rank's experts of layer ``i`` (local) and on the replicated router (gradient all-reduced)."""
        e, o = self.experts[i], self.opt
        kw = dict(lr=o.lr, beta1=o.beta1, beta2=o.beta2, eps=o.eps, weight_decay=o.weight_decay, step=self.step_count)
        gate_grad = self.gate_grad_pad[:self.moe.E].float()
        if self.world > 1:
            dist.all_reduce(gate_grad, group=self.comm.group)     # every rank contributed its tokens' share
        lp = e.low_precision()
        # expert gradients hold the sum over all ranks' tokens already; the loss is a mean over world * T tokens and
        # every rank scaled its loss gradient by 1 / (T * world), so nothing is left to average
        for name, grad in (("gate", gate_grad), ("w13", self.g13), ("w2", self.g2)):
            K.adamw_flat(e.master[name].view(-1), e.m[name].view(-1), e.v[name].view(-1), grad.reshape(-1),
                         lp[name].view(-1) if lp[name].is_contiguous() else None, **kw)
        if not lp["gate"].is_contiguous():
            e.gate_pad[:self.moe.E] = e.master["gate"].to(e.gate_pad.dtype)

    # ------------------------------------------------------------------ step
    def step(self, tokens, targets):
        """One optimizer step; returns the global mean next-token loss. ``last_stats['aux_loss']`` holds the mean
        load-balancing loss over the layers of this rank's forward pass (already part of the gradient)."""
        assert tokens.numel() == self.tokens_per_rank, "the dispatch buffers were sized for tokens_per_rank"
        self.aux_losses = []
        loss = super().step(tokens, targets)
        if self.aux_losses:
            self.last_stats = dict(self.last_stats, aux_loss=torch.stack(self.aux_losses).mean())
        return loss

    # ------------------------------------------------------------------ state
    def state_dict(self, master: bool = True, which: str | None = None) -> dict:
        """The dense tensors as in the base engine plus, per layer, ``layers.i.moe.gate`` [E, d] and the experts of
        ALL ranks ``layers.i.moe.w13`` [E, 2f, d], ``layers.i.moe.w2`` [E, d, f]. Collective when ``world > 1``."""
        out = super().state_dict(master, which)
        for i, e in enumerate(self.experts):
            src = {"m": e.m, "v": e.v}.get(which, e.master if master else e.low_precision())
            out[f"layers.{i}.moe.gate"] = src["gate"].float().clone()
            for name in ("w13", "w2"):
                t = src[name].float().contiguous()
                if self.world > 1:
                    full = torch.empty(self.moe.E, *t.shape[1:], dtype=t.dtype, device=t.device)
                    dist.all_gather_into_tensor(full, t, group=self.comm.group)
                    t = full
                out[f"layers.{i}.moe.{name}"] = t.clone() if t is src[name] else t
        return out

    def shard_state(self) -> dict:
        """The base engine's shards plus this rank's experts (``experts.i.<name>.master / exp_avg / exp_avg_sq``).
        Expert tensors are whole experts, not slices of a flat unit: a checkpoint is read back at the same world size."""
        st = super().shard_state()
        for i, e in enumerate(self.experts):
            for name in ("gate", "w13", "w2"):
                st[f"experts.{i}.{name}.master"] = e.master[name]
                st[f"experts.{i}.{name}.exp_avg"] = e.m[name]
                st[f"experts.{i}.{name}.exp_avg_sq"] = e.v[name]
        return st

    def load_shard_state(self, st: dict) -> None:
        for i, e in enumerate(self.experts):
            key = f"experts.{i}.w13.master"
            if key not in st:
                continue          # a dense-only state (weights handed over by name): the experts keep theirs
            assert st[key].shape == e.master["w13"].shape, "expert shards are tied to the world size they were saved at"
            lp = e.low_precision()
            for name in ("gate", "w13", "w2"):
                e.master[name].copy_(st[f"experts.{i}.{name}.master"])
                e.m[name].copy_(st[f"experts.{i}.{name}.exp_avg"])
                e.v[name].copy_(st[f"experts.{i}.{name}.exp_avg_sq"])
                lp[name].copy_(e.master[name].to(lp[name].dtype))
        super().load_shard_state(st)

    def accumulate(self, tokens, targets):
        raise NotImplementedError("the expert optimizer updates a layer right after its backward pass; gradient "
                                  "accumulation over micro-batches is not wired into it")

    def expert_parameters(self) -> int:
        return sum(v.numel() for e in self.experts for v in e.master.values())
