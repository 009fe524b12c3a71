"""GPT-2 style decoder (ghostflow-nn/src/gpt.rs:37-547): ``GPTConfig`` presets, ``GPTEmbeddings`` (learned token +
position), ``GPTModel``, ``GPTForCausalLM.forward/generate`` and ``GPTForSequenceClassification``.

Deviations from the reference, chosen because the benchmark configurations name the standard architecture:
causal masking (the reference builds GPT from its encoder stack and ignores the mask, gpt.rs:294-318,
transformer.rs:97), pre-LayerNorm blocks by default (``pre_norm=False`` gives the reference's post-LN),
an optionally tied output head (the reference's is untied with bias, gpt.rs:339), a KV cache in ``generate``
and real temperature sampling (the reference is greedy whatever the temperature, gpt.rs:402-422).
"""
from __future__ import annotations

import torch

from .. import ops
from ..nn import init
from ..nn.attention import MultiHeadAttention
from ..nn.layers import Dropout, Embedding, LayerNorm, Linear
from ..nn.module import Module, ModuleList
from ..nn.transformer import FeedForward
from .configs import GPTConfig


class GPTEmbeddings(Module):
    def __init__(self, cfg: GPTConfig):
        super().__init__()
        self.wte = Embedding(cfg.vocab_size, cfg.n_embd)
        self.wpe = Embedding(cfg.n_positions, cfg.n_embd)
        self.drop = Dropout(cfg.dropout)

    def forward(self, ids, start_pos: int = 0):
        S = ids.shape[1]
        pos = torch.arange(start_pos, start_pos + S, device=ids.device)
        return self.drop(self.wte(ids) + self.wpe(pos))


class GPTBlock(Module):
    def __init__(self, cfg: GPTConfig):
        super().__init__()
        self.pre_norm = cfg.pre_norm
        self.ln1 = LayerNorm(cfg.n_embd, cfg.layer_norm_eps)
        self.attn = MultiHeadAttention(cfg.n_embd, cfg.n_head, cfg.dropout, causal=cfg.causal)
        self.ln2 = LayerNorm(cfg.n_embd, cfg.layer_norm_eps)
        self.mlp = FeedForward(cfg.n_embd, cfg.n_inner, cfg.dropout, cfg.activation)
        self.drop = Dropout(cfg.dropout)

    def forward(self, x):
        if self.pre_norm:
            if self.drop.p == 0 or not self.training:
                x = self.attn(self.ln1(x), residual=x)          # residual add fused into the GEMM epilogue
                return self.mlp(self.ln2(x), residual=x)
            x = x + self.drop(self.attn(self.ln1(x)))
            return x + self.drop(self.mlp(self.ln2(x)))
        x = self.ln1(x + self.drop(self.attn(x)))
        return self.ln2(x + self.drop(self.mlp(x)))

    def forward_cached(self, x, cache):
        """One decoding step: ``cache = (k, v)`` tensors ``[B, S_past, H, D]`` or (None, None)."""
        h = self.ln1(x) if self.pre_norm else x
        a, _, k, v = self.attn.forward_with_cache(h, cache[0], cache[1])
        if self.pre_norm:
            x = x + a
            return x + self.mlp(self.ln2(x)), (k, v)
        x = self.ln1(x + a)
        return self.ln2(x + self.mlp(x)), (k, v)


class GPTModel(Module):
    def __init__(self, cfg: GPTConfig):
        super().__init__()
        self.cfg = cfg
        self.embeddings = GPTEmbeddings(cfg)
        self.h = ModuleList([GPTBlock(cfg) for _ in range(cfg.n_layer)])
        self.ln_f = LayerNorm(cfg.n_embd, cfg.layer_norm_eps)

    def forward(self, ids):
        x = self.embeddings(ids)
        for blk in self.h:
            x = blk(x)
        return self.ln_f(x)


class GPTForCausalLM(Module):
    def __init__(self, cfg: GPTConfig):
        super().__init__()
        self.cfg = cfg
        self.transformer = GPTModel(cfg)
        self.lm_head = Linear(cfg.n_embd, cfg.vocab_size, bias=False)
        self.reset_parameters()

    @torch.no_grad()
    def reset_parameters(self):
        for name, p in self.named_parameters():
            if p.dim() >= 2:
                if self.cfg.initializer == "xavier_uniform":
                    init.xavier_uniform(p)
                else:
                    p.normal_(0.0, 0.02)
            elif name.endswith("bias"):
                p.zero_()
            elif "ln" in name or "norm" in name:
                p.fill_(1.0)
        if self.cfg.tie_word_embeddings:
            self.lm_head.weight = self.transformer.embeddings.wte.weight

    def forward(self, ids, labels=None):
        logits = self.lm_head(self.transformer(ids))
        if labels is None:
            return logits
        return ops.cross_entropy(logits.view(-1, logits.shape[-1]), labels.reshape(-1)), logits

    @torch.no_grad()
    def generate(self, ids, max_new_tokens: int, temperature: float = 0.0):
        was_training = self.training
        self.eval()
        t = self.transformer
        x = t.embeddings(ids)
        caches = []
        for blk in t.h:
            x, c = blk.forward_cached(x, (None, None))
            caches.append(c)
        logits = self.lm_head(t.ln_f(x))[:, -1]
        out = [ids]
        pos = ids.shape[1]
        for _ in range(max_new_tokens):
            if temperature and temperature > 0:
                nxt = torch.multinomial(torch.softmax(logits.float() / temperature, -1), 1)
            else:
                nxt = logits.argmax(-1, keepdim=True)
            out.append(nxt)
            if pos >= self.cfg.n_positions:
                break
            x = t.embeddings(nxt, start_pos=pos)
            for i, blk in enumerate(t.h):
                x, caches[i] = blk.forward_cached(x, caches[i])
            logits = self.lm_head(t.ln_f(x))[:, -1]
            pos += 1
        self.train(was_training)
        return torch.cat(out, dim=1)


class GPTForSequenceClassification(Module):
    def __init__(self, cfg: GPTConfig, num_labels: int):
        super().__init__()
        self.transformer = GPTModel(cfg)
        self.score = Linear(cfg.n_embd, num_labels, bias=False)

    def forward(self, ids):
        return self.score(self.transformer(ids)[:, -1])
