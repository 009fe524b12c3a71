"""Tensor-parallel LLaMA inference (prefill + greedy decode with a KV cache) on the ranks of one NVSwitch box.

Megatron-style sequence-parallel layout: between blocks the hidden state is sharded over tokens
(``[tokens / world, hidden]`` per rank); inside a block every rank holds ``heads / world`` attention heads and
``ffn / world`` MLP columns. The two collectives of every half-block are fused into the GEMMs around them:

    RMSNorm(shard) -> [all-gather + GEMM] Wqkv -> RoPE -> attention (local heads) -> [GEMM + reduce-scatter] Wo (+res)
    RMSNorm(shard) -> [all-gather + GEMM] W13  -> SwiGLU                          -> [GEMM + reduce-scatter] W2 (+res)

``linear`` selects how those four products run: ``"fused"`` (bf16, one kernel per product incl. its collective),
``"nccl"`` (bf16, NCCL collective then / before the plain GEMM kernel: the baseline), ``"fp8"`` (e4m3 weights
quantised once per output channel, activations per token, scaled tcgen05 fp8 GEMM, NCCL collectives).
The reference has no tensor parallelism and decodes by recomputing the whole sequence on the CPU
(ghostflow-nn/src/gpt.rs generate loop); the KV cache and the decode attention kernel have no counterpart there.
"""
from __future__ import annotations

import math

import torch
import torch.distributed as dist

from ..models.configs import LLaMAConfig
from ..ops import fp8 as fp8_ops
from ..ops import raw
from ..ops.fused import rope_tables
from .tp import AllGatherGemm, GemmReduceScatter, SymmetricWorkspace


def _world(group):
    if dist.is_available() and dist.is_initialized():
        return dist.get_world_size(group), dist.get_rank(group)
    return 1, 0


class _Linears:
    """The four sharded products of a block for one token count (prefill or decode have their own instance because
    the fused kernels own symmetric buffers sized for the token count)."""

    def __init__(self, tokens, hidden, device, group, mode):
        self.mode, self.group, self.T, self.d = mode, group, tokens, hidden
        self.world, self.rank = _world(group)
        self.device = device
        # decode-sized token counts are latency- and bandwidth-bound: there the weight matrices are streamed by
        # the split-K GEMM and the (tiny) collectives stay separate
        self.fused = self.world > 1 and mode == "fused" and tokens > 256
        if self.fused:
            self.ag = AllGatherGemm(tokens, hidden, device, group)
            self.rs = GemmReduceScatter(tokens, hidden, device, group)

    def column(self, x_shard, w):
        """all_gather(x_shard) @ w^T -> [T, n_local]. ``w``: bf16 [n_local, d] or (q, scale) for fp8."""
        if self.world == 1:
            full = x_shard
        elif self.fused:
            return self.ag(x_shard, w)
        else:
            full = torch.empty(self.T, self.d, dtype=x_shard.dtype, device=self.device)
            dist.all_gather_into_tensor(full, x_shard.contiguous(), group=self.group)
        if self.mode == "fp8":
            xq, xs = fp8_ops.quantize_rows(full, 0)
            return fp8_ops.gemm_fp8(xq, xs, w[0], w[1], 0)
        return raw.gemm(full, False, w, True)

    def row(self, x, w, residual):
        """reduce_scatter(x @ w^T) + residual -> [T / world, d]."""
        if self.fused:
            return self.rs(x, w, residual=residual)
        if self.mode == "fp8":
            xq, xs = fp8_ops.quantize_rows(x, 0)
            part = fp8_ops.gemm_fp8(xq, xs, w[0], w[1], 0)
        else:
            part = raw.gemm(x, False, w, True)
        if self.world == 1:
            return part + residual
        out = torch.empty(self.T // self.world, self.d, dtype=part.dtype, device=self.device)
        dist.reduce_scatter_tensor(out, part, group=self.group)
        return out + residual


class TPLlamaInference:
    """``generate(prompt_ids [B, S], max_new_tokens)`` -> ``[B, max_new_tokens]`` greedy tokens (identical on all ranks).

    ``weights``: a dict of FULL tensors with the names of :class:`ghost_flow_b200.models.llama.LLaMAForCausalLM`
    (every rank slices its part), or None for random weights generated shard by shard on the device."""

    def __init__(self, cfg: LLaMAConfig, batch: int, prompt_len: int, max_new_tokens: int, device, group=None,
                 linear: str = "fused", weights: dict | None = None, seed: int = 0, decode: str = "oneshot"):
        assert linear in ("fused", "nccl", "fp8")
        self.cfg, self.group, self.mode = cfg, group, linear
        self.world, self.rank = _world(group)
        self.device = torch.device(device)
        w = self.world
        self.B, self.S, self.max_len = batch, prompt_len, prompt_len + max_new_tokens
        c = cfg
        assert c.num_attention_heads % w == 0 and c.num_key_value_heads % w == 0 and c.intermediate_size % w == 0
        assert (batch * prompt_len) % w == 0 and batch % w == 0 and c.vocab_size % w == 0
        self.Hq, self.Hkv, self.D, self.F = c.num_attention_heads // w, c.num_key_value_heads // w, c.head_dim, c.intermediate_size // w
        self.V = c.vocab_size // w
        self._load(weights, seed)
        self.pre = _Linears(batch * prompt_len, c.hidden_size, self.device, group, linear)
        self.dec = _Linears(batch, c.hidden_size, self.device, group, linear)
        # Decode with replicated activations: each row-parallel projection is followed by ONE kernel that all-reduces
        # the partial products over peer memory, adds the residual and applies the next RMSNorm, so a layer has two
        # collectives (both fused) instead of four. bf16 weights only; other cases use the sequence-parallel step.
        # ``decode="sp"`` keeps the sequence-parallel step (NCCL all-gather / reduce-scatter around split-K GEMMs).
        self.oneshot = (decode == "oneshot" and self.world > 1 and self.device.type == "cuda" and linear != "fp8"
                        and c.hidden_size <= 8192)
        if self.oneshot:
            d = c.hidden_size
            self.ar_ws = SymmetricWorkspace(2 * batch * d * 2 + 4096, self.device, group or dist.group.WORLD)
            self.ar_partial = [self.ar_ws.alloc(batch * d, torch.bfloat16).view(batch, d) for _ in range(2)]
            self.ar_flags = self.ar_ws.alloc(8, torch.int32)
            import ctypes
            mk = lambda v: (ctypes.c_ulonglong * len(v))(*[int(x) for x in v])  # noqa: E731
            self.ar_partial_ptrs = [mk(self.ar_ws.peer_ptrs(t)) for t in self.ar_partial]
            self.ar_flag_ptrs = mk(self.ar_ws.peer_ptrs(self.ar_flags))
            self.ar_epoch = torch.zeros(1, dtype=torch.int32, device=self.device)
            self.ar_done = torch.zeros(1, dtype=torch.int32, device=self.device)
            self.ar_calls = 0
        self.cos, self.sin = rope_tables(self.max_len, self.D, c.rope_theta, self.device)
        kv = (batch, self.max_len, self.Hkv * self.D)
        self.kcache = [torch.zeros(kv, dtype=torch.bfloat16, device=self.device) for _ in range(c.num_hidden_layers)]
        self.vcache = [torch.zeros(kv, dtype=torch.bfloat16, device=self.device) for _ in range(c.num_hidden_layers)]

    # ------------------------------------------------------------------ weights
    def _maybe_q(self, w):
        if self.mode != "fp8":
            return w.contiguous()
        return fp8_ops.quantize_rows(w.contiguous(), 0)

    def _load(self, weights, seed):
        c, r, w, dev, bf = self.cfg, self.rank, self.world, self.device, torch.bfloat16
        d, D = c.hidden_size, self.D
        Hq_all, Hkv_all = c.num_attention_heads, c.num_key_value_heads
        gen = torch.Generator(device=dev).manual_seed(seed * 1000 + r) if weights is None else None

        def rnd(*shape):
            return (torch.randn(*shape, device=dev, generator=gen, dtype=torch.float32) * c.initializer_range).to(bf)

        def get(name):
            return weights[name].to(dev, bf)

        self.layers = []
        for i in range(c.num_hidden_layers):
            p = f"model.layers.{i}."
            if weights is None:
                wqkv, wo = rnd((self.Hq + 2 * self.Hkv) * D, d), rnd(d, self.Hq * D)
                w13, w2 = rnd(2 * self.F, d), rnd(d, self.F)
                n1 = n2 = torch.ones(d, device=dev, dtype=bf)
            else:
                full = get(p + "attn.wqkv.weight")
                q, k, v = full[:Hq_all * D], full[Hq_all * D:(Hq_all + Hkv_all) * D], full[(Hq_all + Hkv_all) * D:]
                wqkv = torch.cat((q[r * self.Hq * D:(r + 1) * self.Hq * D], k[r * self.Hkv * D:(r + 1) * self.Hkv * D],
                                  v[r * self.Hkv * D:(r + 1) * self.Hkv * D]))
                wo = get(p + "attn.wo.weight")[:, r * self.Hq * D:(r + 1) * self.Hq * D]
                gu = get(p + "mlp.gate_up.weight")
                F_all = c.intermediate_size
                w13 = torch.cat((gu[r * self.F:(r + 1) * self.F], gu[F_all + r * self.F:F_all + (r + 1) * self.F]))
                w2 = get(p + "mlp.down.weight")[:, r * self.F:(r + 1) * self.F]
                n1, n2 = get(p + "attn_norm.weight"), get(p + "ffn_norm.weight")
            self.layers.append({"wqkv": self._maybe_q(wqkv), "wo": self._maybe_q(wo), "w13": self._maybe_q(w13),
                                "w2": self._maybe_q(w2), "n1": n1, "n2": n2})
        if weights is None:
            eg = torch.Generator(device=dev).manual_seed(seed * 1000 + 999)     # replicated tensors: same on all ranks
            self.embed = (torch.randn(c.vocab_size, d, device=dev, generator=eg) * c.initializer_range).to(bf)
            self.norm = torch.ones(d, device=dev, dtype=bf)
            self.lm_head = rnd(self.V, d)
        else:
            self.embed, self.norm = get("model.embed_tokens.weight"), get("model.norm.weight")
            self.lm_head = get("lm_head.weight")[r * self.V:(r + 1) * self.V].contiguous()

    # ------------------------------------------------------------------ one transformer block on a token shard
    def _block(self, lin: _Linears, L, h, i, n_seq, seq_len, pos, dev=None):
        """h: [T / world, d]. Prefill: n_seq sequences of seq_len tokens at position 0; decode: seq_len = 1 at pos.
        ``dev`` (decode inside a CUDA graph): (position as a device tensor [1], lengths [B] int32, the cos and sin
        rows of that position) so that nothing in the step depends on a host value."""
        c, eps = self.cfg, self.cfg.rms_norm_eps
        T = lin.T
        x, _, _ = raw.rmsnorm_fwd(h, L["n1"], eps)
        qkv = lin.column(x, L["wqkv"])                                  # [T, (Hq + 2 Hkv) D]
        HD, KD = self.Hq * self.D, self.Hkv * self.D
        q, k, v = qkv[:, :HD], qkv[:, HD:HD + KD], qkv[:, HD + KD:]
        cos, sin, off = (self.cos, self.sin, pos) if dev is None else (dev[2], dev[3], 0)
        raw.rope_(q.unflatten(1, (self.Hq, self.D)), cos, sin, seq_len, c.rope_interleaved, off)
        raw.rope_(k.unflatten(1, (self.Hkv, self.D)), cos, sin, seq_len, c.rope_interleaved, off)
        kc, vc = self.kcache[i], self.vcache[i]
        if seq_len > 1:
            kc[:, :seq_len].copy_(k.view(n_seq, seq_len, KD))
            vc[:, :seq_len].copy_(v.view(n_seq, seq_len, KD))
            o, _ = raw.attn_fwd(q, k, v, n_seq, seq_len, self.Hq, self.Hkv, self.D, True)
        elif dev is not None:
            kc.index_copy_(1, dev[0], k.reshape(n_seq, 1, KD))
            vc.index_copy_(1, dev[0], v.reshape(n_seq, 1, KD))
            o = raw.attn_decode(q, kc, vc, dev[1], n_seq, self.Hq, self.Hkv, self.D)
        else:
            kc[:, pos].copy_(k)
            vc[:, pos].copy_(v)
            o = raw.attn_decode(q, kc, vc, pos + 1, n_seq, self.Hq, self.Hkv, self.D)
        h = lin.row(o, L["wo"], h)
        x, _, _ = raw.rmsnorm_fwd(h, L["n2"], eps)
        a = raw.swiglu_fwd(lin.column(x, L["w13"]))
        return lin.row(a, L["w2"], h)

    # ------------------------------------------------------------------ decode with replicated activations
    def _ar_norm(self, partial_idx, h, norm_w):
        """(h + sum over ranks of partial, RMSNorm of that) in one kernel; see ``gf_allreduce_residual_rmsnorm``."""
        import ctypes
        from ..ops import _lib
        lib = _lib.cuda_lib()
        if not getattr(lib, "_ar_bound", False):
            P, I, L, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float
            lib.gf_allreduce_residual_rmsnorm.argtypes = [P, P, I, I, P, P, P, P, F, P, P, I, I, L, P, P]
            lib.gf_allreduce_residual_rmsnorm.restype = I
            lib._ar_bound = True
        B, d = h.shape
        h_out, x_out = torch.empty_like(h), torch.empty_like(h)
        _lib.check_rc(lib.gf_allreduce_residual_rmsnorm(
            self.ar_partial_ptrs[partial_idx], self.ar_flag_ptrs, self.world, self.rank, self.ar_epoch.data_ptr(),
            self.ar_done.data_ptr(), h.data_ptr(), norm_w.data_ptr(), self.cfg.rms_norm_eps, h_out.data_ptr(),
            x_out.data_ptr(), B, d, 0, _lib.status_word(self.device).data_ptr(), _lib.stream_ptr()),
            "gf_allreduce_residual_rmsnorm")
        return h_out, x_out

    def _decode_oneshot(self, tokens, pos, dev=None):
        c = self.cfg
        B = self.B
        h = self.embed[tokens]
        x, _, _ = raw.rmsnorm_fwd(h, self.layers[0]["n1"], c.rms_norm_eps)
        HD, KD = self.Hq * self.D, self.Hkv * self.D
        cos, sin, off = (self.cos, self.sin, pos) if dev is None else (dev[2], dev[3], 0)
        for i, L in enumerate(self.layers):
            qkv = raw.gemm(x, False, L["wqkv"], True)
            q, k, v = qkv[:, :HD], qkv[:, HD:HD + KD], qkv[:, HD + KD:]
            raw.rope_(q.unflatten(1, (self.Hq, self.D)), cos, sin, 1, c.rope_interleaved, off)
            raw.rope_(k.unflatten(1, (self.Hkv, self.D)), cos, sin, 1, c.rope_interleaved, off)
            kc, vc = self.kcache[i], self.vcache[i]
            if dev is not None:
                kc.index_copy_(1, dev[0], k.reshape(B, 1, KD))
                vc.index_copy_(1, dev[0], v.reshape(B, 1, KD))
                o = raw.attn_decode(q, kc, vc, dev[1], B, self.Hq, self.Hkv, self.D)
            else:
                kc[:, pos].copy_(k)
                vc[:, pos].copy_(v)
                o = raw.attn_decode(q, kc, vc, pos + 1, B, self.Hq, self.Hkv, self.D)
            par = self.ar_calls & 1
            self.ar_calls += 1
            raw.gemm(o, False, L["wo"], True, out=self.ar_partial[par])
            h, x = self._ar_norm(par, h, L["n2"])
            a = raw.swiglu_fwd(raw.gemm(x, False, L["w13"], True))
            par = self.ar_calls & 1
            self.ar_calls += 1
            raw.gemm(a, False, L["w2"], True, out=self.ar_partial[par])
            nxt = self.layers[i + 1]["n1"] if i + 1 < len(self.layers) else self.norm
            h, x = self._ar_norm(par, h, nxt)
        return x            # already normalised with the final norm

    def _next_tokens(self, last_hidden, normed=False):
        """last_hidden [B, d] (same on all ranks) -> greedy token per sequence through the vocab-parallel head."""
        x = last_hidden if normed else raw.rmsnorm_fwd(last_hidden, self.norm, self.cfg.rms_norm_eps)[0]
        logits = raw.gemm(x, False, self.lm_head, True, out_dtype=torch.float32)
        val, idx = logits.max(1)
        if self.world == 1:
            return idx, logits
        pair = torch.stack((val, (idx + self.rank * self.V).float()), 1)
        allp = torch.empty(self.world, *pair.shape, device=self.device)
        dist.all_gather_into_tensor(allp, pair, group=self.group)
        best = allp[:, :, 0].argmax(0)
        return allp[best, torch.arange(x.shape[0], device=self.device), 1].long(), logits

    @torch.no_grad()
    def prefill(self, ids: torch.Tensor):
        """ids [B, S] -> first generated token per sequence [B]."""
        B, S, w, r, d = self.B, self.S, self.world, self.rank, self.cfg.hidden_size
        T = B * S
        flat = ids.reshape(-1).to(self.device)
        lo, hi = r * T // w, (r + 1) * T // w
        h = self.embed[flat[lo:hi]]
        for i, L in enumerate(self.layers):
            h = self._block(self.pre, L, h, i, B, S, 0)
        # the last token of every sequence lives on exactly one rank: sum of one-hot contributions
        last = torch.zeros(B, d, dtype=torch.float32, device=self.device)
        pos = torch.arange(B, device=self.device) * S + S - 1
        mine = (pos >= lo) & (pos < hi)
        last[mine] = h[pos[mine] - lo].float()
        if w > 1:
            dist.all_reduce(last, group=self.group)
        tok, self.last_logits = self._next_tokens(last.to(torch.bfloat16))
        return tok

    @torch.no_grad()
    def decode_step(self, tokens: torch.Tensor, pos: int, dev=None):
        """tokens [B] at position ``pos`` -> next tokens [B]."""
        B, w, r, d = self.B, self.world, self.rank, self.cfg.hidden_size
        if self.oneshot:
            tok, self.last_logits = self._next_tokens(self._decode_oneshot(tokens, pos, dev), normed=True)
            return tok
        lo, hi = r * B // w, (r + 1) * B // w
        h = self.embed[tokens[lo:hi]]
        for i, L in enumerate(self.layers):
            h = self._block(self.dec, L, h, i, B, 1, pos, dev)
        if w > 1:
            full = torch.empty(B, d, dtype=h.dtype, device=self.device)
            dist.all_gather_into_tensor(full, h.contiguous(), group=self.group)
        else:
            full = h
        tok, self.last_logits = self._next_tokens(full)
        return tok

    # ------------------------------------------------------------------ decode as one CUDA graph
    @torch.no_grad()
    def capture_decode(self):
        """Captures one decode step (all layers, the collectives, sampling, and the bookkeeping that advances the
        position) into a CUDA graph. A step is about 30 launches per layer, so replaying it removes the host from
        the loop. State lives in device tensors: current tokens, position, lengths."""
        dev = self.device
        self.g_tokens = torch.zeros(self.B, dtype=torch.long, device=dev)
        self.g_pos = torch.full((1,), self.S, dtype=torch.long, device=dev)
        self.g_lens = torch.full((self.B,), self.S + 1, dtype=torch.int32, device=dev)

        def step():
            cos, sin = self.cos.index_select(0, self.g_pos), self.sin.index_select(0, self.g_pos)
            nxt = self.decode_step(self.g_tokens, -1, (self.g_pos, self.g_lens, cos, sin))
            self.g_tokens.copy_(nxt)
            self.g_pos.add_(1)
            self.g_lens.add_(1)

        side = torch.cuda.Stream(dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            for _ in range(2):              # warm-up outside capture: lazy allocations, kernel attributes
                step()
        torch.cuda.current_stream(dev).wait_stream(side)
        torch.cuda.synchronize(dev)
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            step()
        return self.graph

    def graph_decode(self, first_tokens: torch.Tensor, start_pos: int, steps: int):
        """Runs ``steps`` captured decode steps from ``first_tokens`` at ``start_pos``; returns [B, steps]."""
        self.g_tokens.copy_(first_tokens)
        self.g_pos.fill_(start_pos)
        self.g_lens.fill_(start_pos + 1)
        out = []
        for _ in range(steps):
            self.graph.replay()
            out.append(self.g_tokens.clone())
        return torch.stack(out, 1)

    @torch.no_grad()
    def generate(self, ids: torch.Tensor, max_new_tokens: int, use_graph: bool = False):
        first = self.prefill(ids)
        if use_graph and self.device.type == "cuda" and max_new_tokens > 1:
            if not hasattr(self, "graph"):
                self.capture_decode()
            rest = self.graph_decode(first, self.S, max_new_tokens - 1)
            return torch.cat((first[:, None], rest), 1)
        out = [first]
        for t in range(1, max_new_tokens):
            out.append(self.decode_step(out[-1], self.S + t - 1))
        return torch.stack(out, 1)
