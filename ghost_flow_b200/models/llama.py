"""LLaMA-family decoder as ``nn.Module`` (autograd path; the hand-scheduled ZeRO-3 engine in
``parallel/zero3.py`` runs the same math with explicit kernels).

Class and preset names follow ghostflow-nn/src/llama.rs:37-552 (``LLaMAConfig``, ``RMSNorm``, ``RotaryEmbedding``,
``SwiGLU``, ``LLaMAAttention``, ``LLaMADecoderLayer``, ``LLaMAModel``, ``LLaMAForCausalLM.forward/generate``).
Deviations from the reference, on purpose: real causal attention with K and V (its attention is a
placeholder that drops them, llama.rs:319-331), grouped-query attention, no biases, a KV cache in
``generate`` (its doc promises one, the code re-runs the whole prefix), N(0, 0.02) initialisation.
"""
from __future__ import annotations

import torch

from .. import ops
from ..nn.layers import Embedding, Linear, RMSNorm
from ..nn.module import Module, ModuleList
from .configs import LLaMAConfig


class LLaMAAttention(Module):
    def __init__(self, cfg: LLaMAConfig, device=None, dtype=None):
        super().__init__()
        self.cfg = cfg
        hd = cfg.head_dim
        self.wqkv = Linear(cfg.hidden_size, (cfg.num_attention_heads + 2 * cfg.num_key_value_heads) * hd, False,
                           device, dtype)
        self.wo = Linear(cfg.num_attention_heads * hd, cfg.hidden_size, False, device, dtype)

    def forward(self, x, cos, sin, residual=None, cache=None, start_pos: int = 0):
        c = self.cfg
        B, S, _ = x.shape
        H, Hk, D = c.num_attention_heads, c.num_key_value_heads, c.head_dim
        qkv = self.wqkv(x).view(B, S, H + 2 * Hk, D)
        q, k, v = ops.split_qkv(qkv, H, Hk)
        q = ops.rope(q, cos, sin, c.rope_interleaved, start_pos)
        k = ops.rope(k, cos, sin, c.rope_interleaved, start_pos)
        if cache is not None:
            # decoding: append to the cache and attend over everything seen so far
            kc, vc = cache
            kc[:, start_pos:start_pos + S] = k
            vc[:, start_pos:start_pos + S] = v
            kernels = x.is_cuda and x.dtype == torch.bfloat16 and D in (64, 128) and not torch.is_grad_enabled()
            if kernels and S == 1:
                # one new token per sequence: the decode kernel streams the cache once (GQA groups share the reads)
                from ..ops import raw

                o = raw.attn_decode(q.reshape(B, H * D), kc.view(B, kc.shape[1], Hk * D), vc.view(B, vc.shape[1], Hk * D),
                                    start_pos + 1, B, H, Hk, D).view(B, 1, H, D)
            elif kernels and start_pos == 0:
                o = ops.flash_attention(q, k, v, causal=True)        # prompt: nothing older than itself to attend to
            else:
                kk, vv = kc[:, :start_pos + S], vc[:, :start_pos + S]
                G = H // Hk
                qf = q.transpose(1, 2).float()
                kf = kk.transpose(1, 2).float().repeat_interleave(G, 1)
                vf = vv.transpose(1, 2).float().repeat_interleave(G, 1)
                s = qf @ kf.transpose(-1, -2) / (D ** 0.5)
                T = start_pos + S
                mask = torch.ones(S, T, dtype=torch.bool, device=x.device).tril(T - S)
                s = s.masked_fill(~mask, float("-inf"))
                o = (torch.softmax(s, -1) @ vf).transpose(1, 2).to(x.dtype)
        else:
            o = ops.flash_attention(q, k, v, causal=True)
        return self.wo(o.reshape(B, S, H * D), residual)


class LLaMADecoderLayer(Module):
    def __init__(self, cfg: LLaMAConfig, device=None, dtype=None):
        super().__init__()
        from ..nn.layers import SwiGLU

        self.attn_norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, device, dtype)
        self.attn = LLaMAAttention(cfg, device, dtype)
        self.ffn_norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, device, dtype)
        self.mlp = SwiGLU(cfg.hidden_size, cfg.intermediate_size, False, device, dtype)

    def forward(self, x, cos, sin, cache=None, start_pos: int = 0):
        x = self.attn(self.attn_norm(x), cos, sin, residual=x, cache=cache, start_pos=start_pos)
        return self.mlp(self.ffn_norm(x), residual=x)


class LLaMAModel(Module):
    def __init__(self, cfg: LLaMAConfig, device=None, dtype=None):
        super().__init__()
        self.cfg = cfg
        self.embed_tokens = Embedding(cfg.vocab_size, cfg.hidden_size, device=device, dtype=dtype)
        self.layers = ModuleList([LLaMADecoderLayer(cfg, device, dtype) for _ in range(cfg.num_hidden_layers)])
        self.norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, device, dtype)
        self._rope = None

    def rope(self, length, device):
        if self._rope is None or self._rope[0].shape[0] < length or self._rope[0].device != torch.device(device):
            n = max(length, self.cfg.max_position_embeddings)
            self._rope = ops.rope_tables(n, self.cfg.head_dim, self.cfg.rope_theta, device)
        return self._rope

    def forward(self, ids, caches=None, start_pos: int = 0):
        S = ids.shape[1]
        cos, sin = self.rope(start_pos + S, ids.device)
        x = self.embed_tokens(ids)
        for i, layer in enumerate(self.layers):
            x = layer(x, cos, sin, None if caches is None else caches[i], start_pos)
        return self.norm(x)


class LLaMAForCausalLM(Module):
    def __init__(self, cfg: LLaMAConfig, device=None, dtype=None):
        super().__init__()
        self.cfg = cfg
        self.model = LLaMAModel(cfg, device, dtype)
        self.lm_head = Linear(cfg.hidden_size, cfg.vocab_size, False, device, dtype)
        self.reset_parameters()

    @torch.no_grad()
    def reset_parameters(self):
        std = self.cfg.initializer_range
        for name, p in self.named_parameters():
            if name.endswith("norm.weight"):
                p.fill_(1.0)
            else:
                p.normal_(0.0, std)
        if self.cfg.tie_word_embeddings:
            self.lm_head.weight = self.model.embed_tokens.weight

    def forward(self, ids, labels=None, caches=None, start_pos: int = 0):
        h = self.model(ids, caches, start_pos)
        logits = self.lm_head(h)
        if labels is None:
            return logits
        return ops.cross_entropy(logits.view(-1, logits.shape[-1]), labels.reshape(-1)), logits

    def new_caches(self, batch: int, max_len: int, device=None, dtype=None):
        c = self.cfg
        p = next(self.parameters())
        shape = (batch, max_len, c.num_key_value_heads, c.head_dim)
        return [(torch.zeros(shape, device=device or p.device, dtype=dtype or p.dtype),
                 torch.zeros(shape, device=device or p.device, dtype=dtype or p.dtype))
                for _ in range(c.num_hidden_layers)]

    @torch.no_grad()
    def generate(self, ids, max_new_tokens: int, temperature: float = 0.0):
        """Greedy (temperature 0) or sampled continuation with a KV cache."""
        B, S = ids.shape
        caches = self.new_caches(B, S + max_new_tokens)
        logits = self.forward(ids, caches=caches, start_pos=0)[:, -1]
        out = [ids]
        pos = S
        for _ in range(max_new_tokens):
            if temperature and temperature > 0:
                nxt = torch.multinomial(torch.softmax(logits.float() / temperature, -1), 1)
            else:
                nxt = logits.argmax(-1, keepdim=True)
            out.append(nxt)
            logits = self.forward(nxt, caches=caches, start_pos=pos)[:, -1]
            pos += 1
        return torch.cat(out, dim=1)

    # names used by the ZeRO engine's state_dict
    def load_engine_state(self, sd: dict):
        """Loads the flat-unit names of ``Zero3LlamaEngine.state_dict()``."""
        own = self.state_dict()
        own["model.embed_tokens.weight"].copy_(sd["embed_tokens.weight"])
        own["model.norm.weight"].copy_(sd["norm.weight"])
        own["lm_head.weight"].copy_(sd["lm_head.weight"])
        for i in range(self.cfg.num_hidden_layers):
            pre = f"model.layers.{i}."
            own[pre + "attn_norm.weight"].copy_(sd[f"layers.{i}.attn_norm"])
            own[pre + "attn.wqkv.weight"].copy_(sd[f"layers.{i}.wqkv"])
            own[pre + "attn.wo.weight"].copy_(sd[f"layers.{i}.wo"])
            own[pre + "ffn_norm.weight"].copy_(sd[f"layers.{i}.ffn_norm"])
            own[pre + "mlp.gate_up.weight"].copy_(sd[f"layers.{i}.w_gate_up"])
            own[pre + "mlp.down.weight"].copy_(sd[f"layers.{i}.w_down"])
