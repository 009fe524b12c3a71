"""Attention layers.

``scaled_dot_product_attention`` (mask semantics 1 = keep, 0 = -inf, ghostflow-nn/src/attention.rs:11-64),
``MultiHeadAttention`` with a KV cache (``forward_with_cache`` returns (out, weights, k_cache, v_cache):
attention.rs:100-146), ``CrossAttention``, and ``FlashAttention`` with the reference's config presets
(ghostflow-nn/src/flash_attention.rs:27-66). Unmasked or causal attention on bf16 CUDA tensors with head_dim
64/128 runs the tcgen05 FlashAttention kernels; everything else uses the explicit softmax path.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn.functional as F

from .. import ops
from .layers import Dropout, Linear
from .module import Module


def scaled_dot_product_attention(q, k, v, mask=None, dropout_p: float = 0.0, training: bool = False, causal=False,
                                 scale=None, return_weights: bool = False):
    """q, k, v: ``[..., S, D]``. ``mask`` broadcasts over scores; entries equal to 0 are masked out."""
    d = q.shape[-1]
    scale = scale if scale is not None else 1.0 / math.sqrt(d)
    scores = torch.matmul(q, k.transpose(-1, -2)) * scale
    if causal:
        Sq, Sk = scores.shape[-2:]
        cm = torch.ones(Sq, Sk, dtype=torch.bool, device=q.device).tril(Sk - Sq)
        scores = scores.masked_fill(~cm, float("-inf"))
    if mask is not None:
        scores = scores.masked_fill(mask == 0, float("-inf"))
    w = torch.softmax(scores.float(), dim=-1).to(q.dtype)
    if dropout_p > 0 and training:
        w = F.dropout(w, dropout_p)
    out = torch.matmul(w, v)
    return (out, w) if return_weights else out


class MultiHeadAttention(Module):
    """Multi-head (optionally grouped-query) attention with fused QKV projection."""

    def __init__(self, embed_dim: int, num_heads: int, dropout: float = 0.0, bias: bool = True,
                 num_kv_heads: int | None = None, causal: bool = False, device=None, dtype=None):
        super().__init__()
        assert embed_dim % num_heads == 0
        self.embed_dim, self.num_heads = embed_dim, num_heads
        self.num_kv_heads = num_kv_heads or num_heads
        self.head_dim = embed_dim // num_heads
        self.causal = causal
        self.qkv = Linear(embed_dim, (num_heads + 2 * self.num_kv_heads) * self.head_dim, bias, device, dtype)
        self.out_proj = Linear(embed_dim, embed_dim, bias, device, dtype)
        self.dropout = dropout

    def _split(self, x):
        B, S, _ = x.shape
        H, Hk, D = self.num_heads, self.num_kv_heads, self.head_dim
        return ops.split_qkv(self.qkv(x).view(B, S, H + 2 * Hk, D), H, Hk)

    def forward(self, x, mask=None, causal: bool | None = None, rope=None, residual=None):
        """x: ``[B, S, E]``. ``rope`` = (cos, sin, interleaved) applies rotary embedding to q and k."""
        causal = self.causal if causal is None else causal
        B, S, _ = x.shape
        q, k, v = self._split(x)
        if rope is not None:
            cos, sin, inter = rope
            q = ops.rope(q, cos, sin, inter)
            k = ops.rope(k, cos, sin, inter)
        if mask is None and not (self.dropout > 0 and self.training):
            o = ops.flash_attention(q, k, v, causal=causal)
        else:
            G = self.num_heads // self.num_kv_heads
            kk = k.repeat_interleave(G, 2) if G > 1 else k
            vv = v.repeat_interleave(G, 2) if G > 1 else v
            o = scaled_dot_product_attention(q.transpose(1, 2), kk.transpose(1, 2), vv.transpose(1, 2), mask,
                                             self.dropout, self.training, causal).transpose(1, 2)
        return self.out_proj(o.reshape(B, S, self.embed_dim), residual)

    def forward_with_cache(self, x, k_cache=None, v_cache=None, mask=None):
        """Incremental decoding: keys/values of ``x`` are appended to the caches (``[B, S_past, Hkv, D]``).
        Returns ``(out, attention_weights, k_cache, v_cache)``."""
        B, S, _ = x.shape
        q, k, v = self._split(x)
        if k_cache is not None:
            k = torch.cat((k_cache, k), dim=1)
            v = torch.cat((v_cache, v), dim=1)
        G = self.num_heads // self.num_kv_heads
        kk = k.repeat_interleave(G, 2) if G > 1 else k
        vv = v.repeat_interleave(G, 2) if G > 1 else v
        o, w = scaled_dot_product_attention(q.transpose(1, 2), kk.transpose(1, 2), vv.transpose(1, 2), mask, 0.0,
                                            False, self.causal, return_weights=True)
        out = self.out_proj(o.transpose(1, 2).reshape(B, S, self.embed_dim))
        return out, w, k, v


class CrossAttention(Module):
    def __init__(self, embed_dim: int, num_heads: int, kv_dim: int | None = None, dropout: float = 0.0,
                 bias: bool = True):
        super().__init__()
        self.embed_dim, self.num_heads, self.head_dim = embed_dim, num_heads, embed_dim // num_heads
        self.q_proj = Linear(embed_dim, embed_dim, bias)
        self.kv_proj = Linear(kv_dim or embed_dim, 2 * embed_dim, bias)
        self.out_proj = Linear(embed_dim, embed_dim, bias)
        self.dropout = dropout

    def forward(self, x, context, mask=None):
        B, S, _ = x.shape
        Sk = context.shape[1]
        H, D = self.num_heads, self.head_dim
        q = self.q_proj(x).view(B, S, H, D).transpose(1, 2)
        kv = self.kv_proj(context).view(B, Sk, 2, H, D)
        k, v = kv[:, :, 0].transpose(1, 2), kv[:, :, 1].transpose(1, 2)
        o = scaled_dot_product_attention(q, k, v, mask, self.dropout, self.training)
        return self.out_proj(o.transpose(1, 2).reshape(B, S, self.embed_dim))


@dataclass
class FlashAttentionConfig:
    block_size_q: int = 64
    block_size_kv: int = 64
    causal: bool = False
    dropout: float = 0.0
    scale: float | None = None

    @classmethod
    def default(cls): return cls()
    @classmethod
    def causal_(cls): return cls(causal=True)
    @classmethod
    def bidirectional(cls): return cls(causal=False)
    @classmethod
    def long_sequence(cls): return cls(block_size_q=128, block_size_kv=128)


FlashAttentionConfig.causal_config = FlashAttentionConfig.causal_


class FlashAttention(Module):
    """Tiled online-softmax attention. ``forward(q, k, v)`` takes ``[B, S, D]`` (single head, like the
    reference) or ``[B, S, H, D]``. On bf16 CUDA with D in {64, 128} this is the tcgen05 kernel; otherwise the
    blocked online-softmax algorithm below (ghostflow-nn/src/flash_attention.rs:122-250), which never
    materialises the full score matrix."""

    def __init__(self, config: FlashAttentionConfig | None = None):
        super().__init__()
        self.config = config or FlashAttentionConfig()

    def forward(self, q, k, v):
        single = q.dim() == 3
        if single:
            q, k, v = q.unsqueeze(2), k.unsqueeze(2), v.unsqueeze(2)
        c = self.config
        D = q.shape[-1]
        if q.is_cuda and q.dtype == torch.bfloat16 and D in (64, 128):
            o = ops.flash_attention(q, k, v, causal=c.causal, scale=c.scale)
        else:
            o = self._tiled(q, k, v)
        return o.squeeze(2) if single else o

    def _tiled(self, q, k, v):
        c = self.config
        B, S, H, D = q.shape
        Sk = k.shape[1]
        scale = c.scale if c.scale is not None else 1.0 / math.sqrt(D)
        qf, kf, vf = (t.float().transpose(1, 2) for t in (q, k, v))
        G = H // kf.shape[1]
        if G > 1:
            kf, vf = kf.repeat_interleave(G, 1), vf.repeat_interleave(G, 1)
        out = torch.zeros_like(qf)
        for qs in range(0, S, c.block_size_q):
            qe = min(qs + c.block_size_q, S)
            qb = qf[:, :, qs:qe]
            m = torch.full(qb.shape[:-1], float("-inf"), device=q.device)
            l = torch.zeros_like(m)
            acc = torch.zeros_like(qb)
            for ks in range(0, Sk, c.block_size_kv):
                if c.causal and ks > qe - 1:
                    break
                ke = min(ks + c.block_size_kv, Sk)
                s = qb @ kf[:, :, ks:ke].transpose(-1, -2) * scale
                if c.causal:
                    qi = torch.arange(qs, qe, device=q.device)[:, None]
                    ki = torch.arange(ks, ke, device=q.device)[None, :]
                    s = s.masked_fill(ki > qi, float("-inf"))
                m_new = torch.maximum(m, s.amax(-1))
                p = torch.exp(s - m_new[..., None])
                alpha = torch.exp(m - m_new)
                l = l * alpha + p.sum(-1)
                acc = acc * alpha[..., None] + p @ vf[:, :, ks:ke]
                m = m_new
            out[:, :, qs:qe] = acc / l[..., None]
        return out.transpose(1, 2).to(q.dtype)

    def memory_usage_ratio(self, seq_len: int) -> float:
        """Tile memory relative to the full score matrix (ghostflow-nn/src/flash_attention.rs:285-293)."""
        c = self.config
        return min(1.0, (c.block_size_q * c.block_size_kv) / float(seq_len * seq_len))
