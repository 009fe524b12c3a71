"""Hand-scheduled ZeRO-3 training engine for LLaMA-family decoders.

One process per GPU. Every unit (the embedding, each decoder layer, the head) is ONE flat bf16
buffer cut into equal shards across the ranks; each rank also holds the fp32 master weights and
Adam moments of its shard only. A step walks the layers with explicit forward and backward
kernels (no autograd graph):

    forward : all-gather(layer i+1) runs on the communication stream while layer i computes
    backward: all-gather(layer i-1) is prefetched; layer i's weight gradients are written by the
              wgrad GEMMs straight into a flat gradient buffer, which is reduce-scattered and fed
              to the fused AdamW on the shard while layer i-1 is already computing

so parameters, gradients and optimizer state are all partitioned (stage 3), at most two gathered
layers and two gradient buffers exist at any time, and the optimizer never sees a full model.

Replaces the reference's in-process simulation: whole-tensor "ownership", reduce-scatter = divide
by world size, all-gather = clone, Adam without bias correction
(ghostflow-nn/src/zero_optimizer.rs:149-195,220-259,262-309).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch
import torch.distributed as dist

from ..models.configs import LLaMAConfig
from ..ops import raw as K
from ..ops.fused import rope_tables


@dataclass
class OptimConfig:
    lr: float = 3e-4
    beta1: float = 0.9
    beta2: float = 0.95
    eps: float = 1e-8
    weight_decay: float = 0.01
    # Global-norm gradient clipping. When set, a step first reduces all gradients (keeping each rank's reduced fp32
    # shard), forms the global norm with one scalar all-reduce, and only then updates, with the clip coefficient
    # folded into the AdamW kernel; a non-finite norm skips the update altogether (the step count does not advance).
    # Without it the update of a layer runs inside the reducer while the backward pass is still going.
    # (The reference scans for inf/nan and skips the step in its GradScaler, ghostflow-nn/src/mixed_precision.rs:115-180,
    # and advertises clipping without implementing it.)
    max_grad_norm: float | None = None


class _Unit:
    """One flat parameter unit and this rank's shard of it."""

    def __init__(self, name, specs, world, rank, device, dtype, align=8, index=0):
        self.name = name
        self.index = index
        self.specs = []  # (pname, offset, shape)
        off = 0
        for pname, shape in specs:
            n = math.prod(shape)
            self.specs.append((pname, off, tuple(shape)))
            off += (n + align - 1) // align * align
        self.numel = off
        quantum = world * 16
        self.padded = (off + quantum - 1) // quantum * quantum
        self.shard_numel = self.padded // world
        self.lo = rank * self.shard_numel
        self.shard = None   # allocated by the engine (from the communicator's arena when it has one)
        self.gred = None    # reduced fp32 gradient shard, only with gradient clipping (allocated on first use)
        self.master = None
        self.m = None
        self.v = None

    def views(self, flat):
        return {p: flat[o:o + math.prod(s)].view(s) for p, o, s in self.specs}


class Comm:
    """Collective plumbing for the engine: NCCL/gloo baseline. ``world == 1`` is a no-op."""

    def __init__(self, group=None):
        self.group = group
        if dist.is_available() and dist.is_initialized():
            self.world = dist.get_world_size(group)
            self.rank = dist.get_rank(group)
            self.backend = dist.get_backend(group)
        else:
            self.world, self.rank, self.backend = 1, 0, "none"

    fused = False

    def reserve(self, nbytes: int) -> None:
        """Hook for communicators that keep weights and gradient buffers in a symmetric arena."""

    def alloc(self, numel: int, dtype, device=None) -> torch.Tensor:
        return torch.zeros(numel, dtype=dtype, device=device)

    def all_gather(self, shard, full):
        if self.world == 1:
            return
        dist.all_gather_into_tensor(full, shard, group=self.group)

    def reduce_scatter(self, full, shard_out):
        """Sum over ranks of ``full`` cut into world pieces; piece ``rank`` lands in ``shard_out``."""
        if self.world == 1:
            return
        if self.backend == "nccl":
            dist.reduce_scatter_tensor(shard_out, full, op=dist.ReduceOp.SUM, group=self.group)
        else:
            tmp = full.float()
            dist.all_reduce(tmp, group=self.group)
            n = shard_out.numel()
            shard_out.copy_(tmp[self.rank * n:(self.rank + 1) * n].to(shard_out.dtype))

    def all_reduce_scalar(self, t):
        if self.world > 1:
            dist.all_reduce(t, group=self.group)
        return t


class _Streams:
    """Compute / communication / optimizer streams (all None on CPU, where everything is serial)."""

    def __init__(self, device):
        self.cuda = device.type == "cuda"
        if self.cuda:
            self.comm = torch.cuda.Stream(device)
            self.opt = torch.cuda.Stream(device)

    def event(self):
        return torch.cuda.Event() if self.cuda else None


class Zero3LlamaEngine:
    """ZeRO-3 trainer for :class:`LLaMAConfig` models (dense decoder, GQA allowed)."""

    def __init__(self, cfg: LLaMAConfig, device, optim: OptimConfig | None = None, group=None, seed: int = 0,
                 dtype=torch.bfloat16, comm: Comm | None = None, persist_gathered: bool | None = None,
                 recompute_activations: bool = False):
        self.cfg = cfg
        # Activation recompute: the forward pass keeps only every layer's input (one [T, d] tensor instead of the
        # eleven tensors a layer saves, about 0.55 GB per layer of the 7 B model at 4096 tokens) and the backward
        # pass runs the layer's forward again right before its backward. The kernels are deterministic, so the
        # step computes the same numbers; it costs one more forward pass per step.
        self.recompute = bool(recompute_activations)
        self.device = torch.device(device)
        self.dtype = dtype
        self.opt = optim or OptimConfig()
        self.comm = comm or Comm(group)
        self.world, self.rank = self.comm.world, self.comm.rank
        self.streams = _Streams(self.device)
        self.step_count = 0
        d, f, v = cfg.hidden_size, cfg.intermediate_size, cfg.vocab_size
        hd = cfg.head_dim
        self.qkv_out = (cfg.num_attention_heads + 2 * cfg.num_key_value_heads) * hd
        layer_specs = self._layer_specs()
        mk = lambda name, specs, idx: _Unit(name, specs, self.world, self.rank, self.device, dtype, index=idx)
        self.embed = mk("embed", [("tok_emb", (v, d))], 0)
        self.layers = [mk(f"layer{i}", layer_specs, i + 1) for i in range(cfg.num_hidden_layers)]
        self.head = mk("head", [("final_norm", (d,)), ("lm_head", (v, d))], cfg.num_hidden_layers + 1)
        self.units = [self.embed, *self.layers, self.head]
        max_padded = max(u.padded for u in self.units)
        esz = torch.empty((), dtype=dtype).element_size()
        # weights shards and the two gradient staging buffers come from the communicator (a symmetric,
        # peer-mapped arena for the fused path; plain device memory otherwise)
        self.comm.reserve(sum((u.shard_numel * esz + 255) // 256 * 256 for u in self.units)
                          + 2 * ((max_padded * esz + 255) // 256 * 256) + 4096)
        for u in self.units:
            u.shard = self.comm.alloc(u.shard_numel, dtype, self.device)
        self.gfull = [self.comm.alloc(max_padded, dtype, self.device) for _ in range(2)]
        self._init_params(seed)
        # Gathered weights. Two rotating buffers are enough for correctness (a layer is gathered again in the
        # backward pass). With ``persist_gathered`` every layer keeps its gathered copy from the forward pass until
        # its backward pass has run, so each layer crosses NVLink once per step instead of twice; parameters,
        # gradients and optimizer state stay partitioned, the copies are a cache that lives inside one step. The
        # cost is one low-precision copy of the layer weights (13 GB for the 7 B model of a 180 GB GPU); by
        # default it is taken when that is at most a quarter of the free device memory.
        self.persist = False
        self.full_layers = None
        if self.world > 1:
            self.full = [torch.empty(max_padded, dtype=dtype, device=self.device) for _ in range(2)]
            self.gshard = torch.empty(max(u.shard_numel for u in self.units), dtype=dtype, device=self.device)
            need = sum(u.padded for u in self.layers) * esz
            if persist_gathered is None:
                if self.device.type == "cuda":
                    free, _ = torch.cuda.mem_get_info(self.device)
                    persist_gathered = need <= free // 4
                else:
                    persist_gathered = True
            if persist_gathered and self.layers:
                self.persist = True
                self.full_layers = [torch.empty(u.padded, dtype=dtype, device=self.device) for u in self.layers]
        self._rope = None
        self.last_stats = {}
        self.skipped_steps = 0
        self._sumsq = torch.zeros(1, dtype=torch.float32, device=self.device)
        self._micro = 0            # micro-batches since the last optimizer update (gradient accumulation)
        self._applying = True      # False while a micro-batch of accumulate() runs
        self._gred_tmp = None
        # kernel status word of the previous steps, copied to pinned memory without stalling the stream
        self._status_host = None
        self._status_event = None

    def _layer_specs(self):
        """Named tensors of one decoder layer's flat unit (subclasses with another MLP override this)."""
        c = self.cfg
        d, f, hd = c.hidden_size, c.intermediate_size, c.head_dim
        return [("attn_norm", (d,)), ("wqkv", (self.qkv_out, d)), ("wo", (d, c.num_attention_heads * hd)),
                ("ffn_norm", (d,)), ("w_gate_up", (2 * f, d)), ("w_down", (d, f))]

    # ------------------------------------------------------------------ init
    def _init_params(self, seed):
        """N(0, std) weights, unit norm gains; each unit is generated whole from its own seed (so every
        world size sees the same model) and only this rank's slice is kept."""
        std = self.cfg.initializer_range
        for ui, u in enumerate(self.units):
            gen = torch.Generator(device=self.device)
            gen.manual_seed(seed * 100003 + ui)
            flat = torch.zeros(u.padded, dtype=torch.float32, device=self.device)
            for pname, off, shape in u.specs:
                n = math.prod(shape)
                if pname.endswith("norm"):
                    flat[off:off + n] = 1.0
                else:
                    flat[off:off + n].normal_(0.0, std, generator=gen)
            sl = flat[u.lo:u.lo + u.shard_numel]
            u.master = sl.clone()
            u.shard.copy_(sl.to(self.dtype))
            u.m = torch.zeros_like(u.master)
            u.v = torch.zeros_like(u.master)
            del flat

    def load_unit(self, unit: _Unit, named: dict):
        """Overwrites a unit from full named tensors (used by tests and checkpoint loading)."""
        flat = torch.zeros(unit.padded, dtype=torch.float32, device=self.device)
        for pname, off, shape in unit.specs:
            flat[off:off + math.prod(shape)] = named[pname].to(self.device, torch.float32).reshape(-1)
        sl = flat[unit.lo:unit.lo + unit.shard_numel]
        unit.master.copy_(sl)
        unit.shard.copy_(sl.to(self.dtype))

    def gather_unit(self, unit: _Unit, master: bool = False, which: str | None = None) -> dict:
        """Full named tensors of a unit on every rank: the bf16 weights, the fp32 master copy (``master``), or
        with ``which`` = "m" / "v" the first / second Adam moment."""
        src = {"m": unit.m, "v": unit.v}[which] if which else (unit.master if master else unit.shard)
        if self.world == 1:
            flat = src
        else:
            flat = torch.empty(unit.padded, dtype=src.dtype, device=self.device)
            self.comm.all_gather(src.contiguous(), flat)
        return {k: v.clone() for k, v in unit.views(flat).items()}

    # ------------------------------------------------------------------ gather / scatter scheduling
    def _gather_async(self, unit, slot):
        """Starts the all-gather of ``unit`` into rotating buffer ``slot`` (an int) or into the given tensor;
        returns (flat_full, event)."""
        if self.world == 1:
            return unit.shard, None
        st = self.streams
        full = (self.full[slot] if isinstance(slot, int) else slot)[:unit.padded]
        if st.cuda:
            st.comm.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(st.comm):
                if self.comm.fused:
                    self.comm.all_gather_unit(unit, unit.index, full)
                else:
                    self.comm.all_gather(unit.shard, full)
                ev = st.event()
                ev.record(st.comm)
            return full, ev
        self.comm.all_gather(unit.shard, full)
        return full, None

    def _wait(self, ev):
        if ev is not None:
            torch.cuda.current_stream().wait_event(ev)

    def _acquire_grad_slot(self, slot, local_event):
        """Before the first write into gradient buffer ``slot``: this rank's previous reduce/update of it is
        done (event) and, on the peer-memory path, every peer has finished reading it (flags)."""
        self._wait(local_event)
        if self.comm.fused:
            self.comm.wait_grad_slot_free(slot)

    def _reduce_and_update(self, unit, slot):
        """Gradient reduce-scatter + AdamW on this rank's shard, off the compute stream.
        Returns an event that marks when gradient buffer ``slot`` may be overwritten. With gradient clipping the
        update is deferred: only the reduction runs here (see :meth:`_finish_clipped_step`)."""
        st = self.streams
        g_full = self.gfull[slot][:unit.padded]
        o = self.opt
        kw = dict(lr=o.lr, beta1=o.beta1, beta2=o.beta2, eps=o.eps, weight_decay=o.weight_decay,
                  step=self.step_count)
        # deferred: with clipping, and for every micro-batch of an accumulated step (the first one overwrites the
        # accumulator, the later ones add to it; the norm of the sum is then taken in _finish_clipped_step)
        accumulating = self._micro > 1 or not self._applying
        deferred = o.max_grad_norm is not None or accumulating
        first = self._micro == 1

        def run():
            if deferred:
                if unit.gred is None:
                    unit.gred = torch.zeros(unit.shard_numel, dtype=torch.float32, device=self.device)
                if self.comm.fused:
                    if first:
                        self.comm.reduce_only(unit, unit.index, g_full, slot, unit.gred, self._sumsq)
                    else:
                        if self._gred_tmp is None or self._gred_tmp.numel() < unit.shard_numel:
                            self._gred_tmp = torch.empty(max(u.shard_numel for u in self.units), dtype=torch.float32,
                                                         device=self.device)
                        tmp = self._gred_tmp[:unit.shard_numel]
                        self.comm.reduce_only(unit, unit.index, g_full, slot, tmp, self._sumsq)
                        unit.gred.add_(tmp)
                    return
                if self.world == 1:
                    new = g_full[:unit.shard_numel].float()
                else:
                    g = self.gshard[:unit.shard_numel]
                    self.comm.reduce_scatter(g_full, g)
                    new = g.float()
                if first:
                    unit.gred.copy_(new)
                    self._sumsq.add_(unit.gred.square().sum())
                else:
                    unit.gred.add_(new)
                return
            if self.comm.fused:
                self.comm.reduce_scatter_adamw(unit, unit.index, g_full, slot, **kw)
                return
            if self.world == 1:
                g = g_full
            else:
                g = self.gshard[:unit.shard_numel]
                self.comm.reduce_scatter(g_full, g)
            K.adamw_flat(unit.master, unit.m, unit.v, g, unit.shard, **kw)

        if self.comm.fused:
            self.comm.grads_ready(slot)   # compute stream: my gradients for this buffer are complete
        if st.cuda:
            side = st.opt if (self.world == 1 or self.comm.fused) else st.comm
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                run()
                ev = st.event()
                ev.record(side)
            return ev
        run()
        return None

    def _finish_clipped_step(self):
        """Second half of a step with ``max_grad_norm``: global norm from the per-shard sums of squares (one scalar
        all-reduce), clip coefficient, AdamW on every shard. Returns False when the norm was not finite and the
        update was skipped."""
        o = self.opt
        if self.streams.cuda:
            torch.cuda.current_stream().wait_stream(self.streams.opt)
            torch.cuda.current_stream().wait_stream(self.streams.comm)
        n_micro = max(1, self._micro)
        if n_micro > 1:
            # the per-unit sums of squares were taken per micro-batch: take the norm of the accumulated mean instead
            total = torch.stack([u.gred.square().sum() for u in self.units]).sum().reshape(1) / float(n_micro) ** 2
        else:
            total = self._sumsq.clone()
        self._sumsq.zero_()
        if o.max_grad_norm is None:
            # accumulation without clipping: no norm, no host read
            self.last_stats = {"micro_batches": n_micro}
            for u in self.units:
                K.adamw_flat(u.master, u.m, u.v, u.gred, u.shard, lr=o.lr, beta1=o.beta1, beta2=o.beta2, eps=o.eps,
                             weight_decay=o.weight_decay, step=self.step_count, grad_scale=1.0 / n_micro)
                if self.comm.fused:
                    self.comm.publish_version(u.index)
            return True
        if self.world > 1:
            self.comm.all_reduce_scalar(total)
        norm = float(total.sqrt())                      # one host read per step: the decision to skip is the host's
        finite = math.isfinite(norm)
        coef = (min(1.0, o.max_grad_norm / (norm + 1e-6)) if finite else 0.0) / n_micro
        self.last_stats = {"grad_norm": norm, "clip_coef": coef * n_micro, "skipped": not finite,
                           "micro_batches": n_micro}
        if not finite:
            self.step_count -= 1                        # bias correction continues from the last applied step
            self.skipped_steps += 1
            return False
        for u in self.units:
            K.adamw_flat(u.master, u.m, u.v, u.gred, u.shard, lr=o.lr, beta1=o.beta1, beta2=o.beta2, eps=o.eps,
                         weight_decay=o.weight_decay, step=self.step_count, grad_scale=coef)
            if self.comm.fused:
                self.comm.publish_version(u.index)
        return True

    # ------------------------------------------------------------------ layer math
    def _rope_tables(self, S):
        if self._rope is None or self._rope[0].shape[0] < S:
            self._rope = rope_tables(S, self.cfg.head_dim, self.cfg.rope_theta, self.device)
        return self._rope

    def _attn_fwd(self, w, x, B, S):
        """x -> x + attention(rmsnorm(x)); returns (x2, saved)."""
        c = self.cfg
        Hq, Hkv, hd = c.num_attention_heads, c.num_key_value_heads, c.head_dim
        cos, sin = self._rope_tables(S)
        h1, rstd1, _ = K.rmsnorm_fwd(x, w["attn_norm"], c.rms_norm_eps)
        qkv = K.gemm(h1, False, w["wqkv"], True)
        T = x.shape[0]
        K.rope_(qkv.view(T, Hq + 2 * Hkv, hd)[:, :Hq + Hkv], cos, sin, S, c.rope_interleaved)
        q, k, v = qkv[:, :Hq * hd], qkv[:, Hq * hd:(Hq + Hkv) * hd], qkv[:, (Hq + Hkv) * hd:]
        attn, lse = K.attn_fwd(q, k, v, B, S, Hq, Hkv, hd, causal=True)
        x2 = K.gemm(attn, False, w["wo"], True, residual=x)
        return x2, (x, rstd1, h1, qkv, attn, lse)

    def _attn_bwd(self, w, g, saved, dx2, B, S):
        """Backward of :meth:`_attn_fwd`: ``dx2`` is the gradient of its output (residual branch included);
        writes the weight gradients into ``g`` and returns the gradient of its input."""
        c = self.cfg
        Hq, Hkv, hd = c.num_attention_heads, c.num_key_value_heads, c.head_dim
        cos, sin = self._rope_tables(S)
        x, rstd1, h1, qkv, attn, lse = saved
        T = x.shape[0]
        dattn = K.gemm(dx2, False, w["wo"], False)
        K.gemm(dx2, True, attn, False, out=g["wo"])
        dqkv = torch.empty_like(qkv)
        q, k, v = qkv[:, :Hq * hd], qkv[:, Hq * hd:(Hq + Hkv) * hd], qkv[:, (Hq + Hkv) * hd:]
        dq, dk, dv = dqkv[:, :Hq * hd], dqkv[:, Hq * hd:(Hq + Hkv) * hd], dqkv[:, (Hq + Hkv) * hd:]
        K.attn_bwd(q, k, v, attn, dattn, lse, dq, dk, dv, B, S, Hq, Hkv, hd, causal=True)
        K.rope_(dqkv.view(T, Hq + 2 * Hkv, hd)[:, :Hq + Hkv], cos, sin, S, c.rope_interleaved, backward=True)
        dh1 = K.gemm(dqkv, False, w["wqkv"], False)
        K.gemm(dqkv, True, h1, False, out=g["wqkv"])
        dx, _ = K.rmsnorm_bwd(x, w["attn_norm"], dh1, rstd1, dres=dx2, dw_out=g["attn_norm"])
        return dx

    def _layer_fwd(self, w, x, B, S, layer_index: int = 0):
        c = self.cfg
        x2, sa = self._attn_fwd(w, x, B, S)
        h2, rstd2, _ = K.rmsnorm_fwd(x2, w["ffn_norm"], c.rms_norm_eps)
        gu = K.gemm(h2, False, w["w_gate_up"], True)
        act = K.swiglu_fwd(gu)
        out = K.gemm(act, False, w["w_down"], True, residual=x2)
        return out, (sa, x2, rstd2, h2, gu, act)

    def _layer_bwd(self, w, g, saved, dout, B, S, layer_index: int = 0):
        sa, x2, rstd2, h2, gu, act = saved
        # MLP
        dact = K.gemm(dout, False, w["w_down"], False)
        K.gemm(dout, True, act, False, out=g["w_down"])
        dgu = K.swiglu_bwd(gu, dact)
        del dact
        dh2 = K.gemm(dgu, False, w["w_gate_up"], False)
        K.gemm(dgu, True, h2, False, out=g["w_gate_up"])
        del dgu
        dx2, _ = K.rmsnorm_bwd(x2, w["ffn_norm"], dh2, rstd2, dres=dout, dw_out=g["ffn_norm"])
        return self._attn_bwd(w, g, sa, dx2, B, S)

    # ------------------------------------------------------------------ one training step
    def accumulate(self, tokens: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
        """Forward and backward of one micro-batch WITHOUT an optimizer step: every unit's gradient is reduced over
        the ranks as usual and added to this rank's fp32 shard accumulator. The next :meth:`step` adds its own
        micro-batch and applies AdamW to the mean over all micro-batches since the last update. Returns this
        micro-batch's global mean loss."""
        return self.step(tokens, targets, _apply=False)

    def step(self, tokens: torch.Tensor, targets: torch.Tensor, _apply: bool = True) -> torch.Tensor:
        """One optimizer step on this rank's micro-batch ``tokens/targets [B, S]`` (int64, on device).
        Returns the global mean loss as a 0-d fp32 tensor on the device."""
        c = self.cfg
        B, S = tokens.shape
        T = B * S
        self._poll_status(force=(self.step_count % 8 == 7))
        self._micro += 1
        self._applying = _apply
        if _apply:
            self.step_count += 1
        L = len(self.layers)
        tok = tokens.reshape(-1)
        tgt = targets.reshape(-1)

        # ---------------- forward
        # Gathered-weight buffers: embedding -> 0; layer i -> its own buffer when the gathered copies persist, else
        # rotating buffer (i + 1) % 2; head -> 1 when they persist, else (L - 1) % 2 (or 1 when L == 0).
        # _gather_async makes the communication stream wait for everything already submitted on the
        # compute stream, i.e. for the previous user of the buffer, and no more.
        def layer_buf(i):
            return self.full_layers[i] if self.persist else (i + 1) % 2

        head_buf = 1 if (self.persist or L == 0) else (L - 1) % 2
        emb_full, ev = self._gather_async(self.embed, 0)
        nxt = self._gather_async(self.layers[0], layer_buf(0)) if L else self._gather_async(self.head, head_buf)
        self._wait(ev)
        x = self.embed.views(emb_full)["tok_emb"].index_select(0, tok)
        saved = []
        w_full = None
        for i, unit in enumerate(self.layers):
            w_full, ev = nxt
            nxt = (self._gather_async(self.layers[i + 1], layer_buf(i + 1)) if i + 1 < L
                   else self._gather_async(self.head, head_buf))
            self._wait(ev)
            x_in = x
            x, sv = self._layer_fwd(unit.views(w_full), x, B, S, i)
            saved.append(x_in if self.recompute else sv)
        head_full, ev = nxt
        self._wait(ev)
        hw = self.head.views(head_full)
        hF, rstdF, _ = K.rmsnorm_fwd(x, hw["final_norm"], c.rms_norm_eps)
        logits = K.gemm(hF, False, hw["lm_head"], True)
        loss = K.xent_fwd_bwd(logits, tgt, grad_scale=1.0 / (T * self.world)) * self.world  # local mean

        # ---------------- backward
        grad_free = [None, None]   # events: gradient buffer slot may be overwritten
        gslot = 0
        self._acquire_grad_slot(gslot, None)
        gh = self.head.views(self.gfull[gslot][:self.head.padded])
        dhF = K.gemm(logits, False, hw["lm_head"], False)
        K.gemm(logits, True, hF, False, out=gh["lm_head"])
        del logits
        dx, _ = K.rmsnorm_bwd(x, hw["final_norm"], dhF, rstdF, dw_out=gh["final_norm"])
        grad_free[gslot] = self._reduce_and_update(self.head, gslot)
        # the last layer's weights are still gathered in their buffer from the forward pass; with persistent
        # copies so are all the others
        nxt = (w_full, None)
        for i in range(L - 1, -1, -1):
            unit = self.layers[i]
            gslot = 1 - gslot
            w_full, ev = nxt
            if i > 0:
                nxt = ((self.full_layers[i - 1][:self.layers[i - 1].padded], None) if self.persist
                       else self._gather_async(self.layers[i - 1], i % 2))
            self._wait(ev)
            self._acquire_grad_slot(gslot, grad_free[gslot])
            g = unit.views(self.gfull[gslot][:unit.padded])
            sv = saved.pop()
            if self.recompute:
                _, sv = self._layer_fwd(unit.views(w_full), sv, B, S, i)
            dx = self._layer_bwd(unit.views(w_full), g, sv, dx, B, S, i)
            grad_free[gslot] = self._reduce_and_update(unit, gslot)
        # embedding gradient: scatter-add of dx rows
        gslot = 1 - gslot
        self._acquire_grad_slot(gslot, grad_free[gslot])
        ge = self.embed.views(self.gfull[gslot][:self.embed.padded])["tok_emb"]
        ge.zero_()
        ge.index_add_(0, tok, dx)
        grad_free[gslot] = self._reduce_and_update(self.embed, gslot)
        for e in grad_free:
            self._wait(e)
        if _apply and (self.opt.max_grad_norm is not None or self._micro > 1):
            self._finish_clipped_step()
        if _apply:
            self._micro = 0
        if self.world > 1:
            loss = self.comm.all_reduce_scalar(loss.clone()) / self.world
        self._post_status()
        return loss

    # ------------------------------------------------------------------ learning-rate hook
    def get_lr(self) -> float:
        return self.opt.lr

    def set_lr(self, lr: float) -> None:
        """The engine can be handed to a learning-rate scheduler in place of an optimizer
        (``CosineAnnealingLR(engine, ...)``): schedulers only need ``get_lr`` / ``set_lr``."""
        self.opt.lr = float(lr)

    # ------------------------------------------------------------------ kernel status
    def _post_status(self):
        """Queues a copy of the per-device kernel status word (bounded waits that ran out write a code there)
        into pinned host memory behind this step's kernels; costs no synchronisation."""
        if self.device.type != "cuda":
            return
        from ..ops import _lib

        if self._status_host is None:
            self._status_host = torch.zeros(8, dtype=torch.int32).pin_memory()
            self._status_event = torch.cuda.Event()
        self._status_host.copy_(_lib.status_word(self.device), non_blocking=True)
        self._status_event.record()

    def _poll_status(self, force: bool = False):
        """Raises :class:`KernelStatusError` if an earlier step recorded an expired wait (a peer flag that never
        arrived, a pipeline stage that never filled). Reads the copy posted by the previous step when it has landed;
        ``force`` waits for it (done every eighth step, so that a step on stale data is noticed soon)."""
        if self._status_event is None:
            return
        if not force and not self._status_event.query():
            return
        self._status_event.synchronize()
        code = int(self._status_host[0])
        if code != 0:
            from ..ops import _lib

            _lib.check_status(self.device)   # raises with the code's meaning and clears the word

    def check_status(self):
        """Synchronises and raises if any kernel of the steps so far recorded an error code."""
        if self.device.type == "cuda":
            from ..ops import _lib

            _lib.check_status(self.device)

    # ------------------------------------------------------------------ inference-style forward (no grad state)
    @torch.no_grad()
    def forward_logits(self, tokens: torch.Tensor) -> torch.Tensor:
        """Logits ``[B, S, vocab]`` with the current weights (gathers one unit at a time, no prefetch)."""
        B, S = tokens.shape
        emb_full, ev = self._gather_async(self.embed, 0)
        self._wait(ev)
        x = self.embed.views(emb_full)["tok_emb"].index_select(0, tokens.reshape(-1))
        slot = 1
        for unit in self.layers:
            w_full, ev = self._gather_async(unit, slot)
            self._wait(ev)
            x, _ = self._layer_fwd(unit.views(w_full), x, B, S, self.layers.index(unit))
            slot = 1 - slot
        head_full, ev = self._gather_async(self.head, slot)
        self._wait(ev)
        hw = self.head.views(head_full)
        hF, _, _ = K.rmsnorm_fwd(x, hw["final_norm"], self.cfg.rms_norm_eps)
        return K.gemm(hF, False, hw["lm_head"], True).view(B, S, -1)

    # ------------------------------------------------------------------ state
    def state_dict(self, master: bool = True, which: str | None = None) -> dict:
        """Full (gathered) named tensors with PyTorch-style dotted names (``which`` = "m" / "v": Adam moments)."""
        out = {}
        out["embed_tokens.weight"] = self.gather_unit(self.embed, master, which)["tok_emb"]
        for i, u in enumerate(self.layers):
            for k, v in self.gather_unit(u, master, which).items():
                out[f"layers.{i}.{k}"] = v
        h = self.gather_unit(self.head, master, which)
        out["norm.weight"] = h["final_norm"]
        out["lm_head.weight"] = h["lm_head"]
        return out

    def _unit_named(self, unit: _Unit, full: dict) -> dict:
        if unit is self.embed:
            return {"tok_emb": full["embed_tokens.weight"]}
        if unit is self.head:
            return {"final_norm": full["norm.weight"], "lm_head": full["lm_head.weight"]}
        i = self.layers.index(unit)
        return {p: full[f"layers.{i}.{p}"] for p, _, _ in unit.specs}

    def load_full_state(self, params: dict, exp_avg: dict | None = None, exp_avg_sq: dict | None = None,
                        step: int = 0) -> None:
        """Restores the engine from full named fp32 tensors (as :meth:`state_dict` returns them): every rank
        keeps its own slice of weights and, when given, of the Adam moments. Collective when ``world > 1``."""
        st = {"step": step}
        for u in self.units:
            for key, full in (("master", params), ("exp_avg", exp_avg), ("exp_avg_sq", exp_avg_sq)):
                if full is None:
                    st[f"{u.name}.{key}"] = torch.zeros(u.shard_numel, dtype=torch.float32, device=self.device)
                    continue
                flat = torch.zeros(u.padded, dtype=torch.float32)
                for pname, off, shape in u.specs:
                    flat[off:off + math.prod(shape)] = self._unit_named(u, full)[pname].to(torch.float32).reshape(-1)
                st[f"{u.name}.{key}"] = flat[u.lo:u.lo + u.shard_numel].to(self.device)
        self.load_shard_state(st)

    def shard_state(self) -> dict:
        """This rank's shards (weights, master, moments) for sharded checkpoints."""
        st = {"step": self.step_count, "world": self.world, "rank": self.rank}
        for u in self.units:
            st[f"{u.name}.master"] = u.master
            st[f"{u.name}.exp_avg"] = u.m
            st[f"{u.name}.exp_avg_sq"] = u.v
        return st

    def load_shard_state(self, st: dict) -> None:
        """Restores this rank's shards (fp32 master, moments) and the step count; the low-precision shard is
        recomputed from the master copy. Collective when ``world > 1``: no rank returns before every rank has
        its new weights in place, because the next step's gathers read the peers' shards directly."""
        self.step_count = int(st["step"])
        for u in self.units:
            u.master.copy_(st[f"{u.name}.master"])
            u.m.copy_(st[f"{u.name}.exp_avg"])
            u.v.copy_(st[f"{u.name}.exp_avg_sq"])
            u.shard.copy_(u.master.to(self.dtype))
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)
        if self.world > 1:
            dist.barrier(group=self.comm.group)

    def flat_layout(self) -> dict:
        """Per unit: logical length, padded length, shard length and this rank's offset in the flat unit
        (what a sharded checkpoint needs to be cut again for another world size)."""
        return {u.name: {"numel": u.numel, "padded": u.padded, "shard_numel": u.shard_numel, "lo": u.lo}
                for u in self.units}

    def memory_summary(self) -> dict:
        per_rank = sum(u.shard_numel for u in self.units)
        return {"params_total": sum(u.numel for u in self.units), "shard_elems": per_rank,
                "bytes_weights_bf16": per_rank * 2, "bytes_optimizer_fp32": per_rank * 12}
