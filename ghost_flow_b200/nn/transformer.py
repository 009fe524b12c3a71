"""Transformer building blocks (ghostflow-nn/src/transformer.rs:11-439): ``FeedForward`` (GELU by default),
encoder / decoder layers with a ``pre_norm`` switch (the reference defaults to post-LN), ``TransformerEncoder``
(adds a final LayerNorm like the reference, transformer.rs:240-243), sinusoidal ``PositionalEncoding`` and
``RotaryEmbedding.apply(q, k, start_pos)`` (half-split pairing, theta 1e4)."""
from __future__ import annotations

import math

import torch

from .. import ops
from .attention import CrossAttention, MultiHeadAttention
from .layers import GELU, Dropout, LayerNorm, Linear, ReLU, SiLU
from .module import Module, ModuleList

_ACTS = {"gelu": GELU, "relu": ReLU, "silu": SiLU}


class FeedForward(Module):
    def __init__(self, d_model: int, d_ff: int, dropout: float = 0.1, activation: str = "gelu", bias: bool = True):
        super().__init__()
        self.fc1 = Linear(d_model, d_ff, bias)
        self.act = _ACTS[activation]()
        self.drop = Dropout(dropout)
        self.fc2 = Linear(d_ff, d_model, bias)

    def forward(self, x, residual=None):
        return self.fc2(self.drop(self.act(self.fc1(x))), residual)


class TransformerEncoderLayer(Module):
    def __init__(self, d_model: int, nhead: int, dim_feedforward: int = 2048, dropout: float = 0.1,
                 pre_norm: bool = False, activation: str = "gelu", causal: bool = False, eps: float = 1e-5):
        super().__init__()
        self.pre_norm = pre_norm
        self.self_attn = MultiHeadAttention(d_model, nhead, dropout, causal=causal)
        self.ff = FeedForward(d_model, dim_feedforward, dropout, activation)
        self.norm1 = LayerNorm(d_model, eps)
        self.norm2 = LayerNorm(d_model, eps)
        self.drop = Dropout(dropout)

    @classmethod
    def with_config(cls, d_model, nhead, dim_feedforward, dropout, pre_norm):
        return cls(d_model, nhead, dim_feedforward, dropout, pre_norm)

    def forward(self, x, mask=None):
        if self.pre_norm:
            x = x + self.drop(self.self_attn(self.norm1(x), mask))
            return x + self.drop(self.ff(self.norm2(x)))
        x = self.norm1(x + self.drop(self.self_attn(x, mask)))
        return self.norm2(x + self.drop(self.ff(x)))

    forward_with_mask = forward


class TransformerDecoderLayer(Module):
    def __init__(self, d_model: int, nhead: int, dim_feedforward: int = 2048, dropout: float = 0.1,
                 pre_norm: bool = False, activation: str = "gelu"):
        super().__init__()
        self.pre_norm = pre_norm
        self.self_attn = MultiHeadAttention(d_model, nhead, dropout, causal=True)
        self.cross_attn = CrossAttention(d_model, nhead, dropout=dropout)
        self.ff = FeedForward(d_model, dim_feedforward, dropout, activation)
        self.norm1, self.norm2, self.norm3 = LayerNorm(d_model), LayerNorm(d_model), LayerNorm(d_model)
        self.drop = Dropout(dropout)

    def forward(self, x, memory, tgt_mask=None, memory_mask=None):
        if self.pre_norm:
            x = x + self.drop(self.self_attn(self.norm1(x), tgt_mask))
            x = x + self.drop(self.cross_attn(self.norm2(x), memory, memory_mask))
            return x + self.drop(self.ff(self.norm3(x)))
        x = self.norm1(x + self.drop(self.self_attn(x, tgt_mask)))
        x = self.norm2(x + self.drop(self.cross_attn(x, memory, memory_mask)))
        return self.norm3(x + self.drop(self.ff(x)))


class TransformerEncoder(Module):
    def __init__(self, d_model: int, nhead: int, dim_feedforward: int, num_layers: int, dropout: float = 0.1,
                 pre_norm: bool = False, activation: str = "gelu", causal: bool = False, final_norm: bool = True):
        super().__init__()
        self.layers = ModuleList([
            TransformerEncoderLayer(d_model, nhead, dim_feedforward, dropout, pre_norm, activation, causal)
            for _ in range(num_layers)])
        self.norm = LayerNorm(d_model) if final_norm else None

    def forward(self, x, mask=None):
        for layer in self.layers:
            x = layer(x, mask)
        return self.norm(x) if self.norm is not None else x

    forward_with_mask = forward


class TransformerDecoder(Module):
    def __init__(self, d_model: int, nhead: int, dim_feedforward: int, num_layers: int, dropout: float = 0.1,
                 pre_norm: bool = False):
        super().__init__()
        self.layers = ModuleList([TransformerDecoderLayer(d_model, nhead, dim_feedforward, dropout, pre_norm)
                                  for _ in range(num_layers)])
        self.norm = LayerNorm(d_model)

    def forward(self, x, memory, tgt_mask=None, memory_mask=None):
        for layer in self.layers:
            x = layer(x, memory, tgt_mask, memory_mask)
        return self.norm(x)


class PositionalEncoding(Module):
    """Sinusoidal table added to the input (ghostflow-nn/src/transformer.rs:294-350)."""

    def __init__(self, d_model: int, max_len: int = 5000, dropout: float = 0.0):
        super().__init__()
        pos = torch.arange(max_len, dtype=torch.float32).unsqueeze(1)
        div = torch.exp(torch.arange(0, d_model, 2, dtype=torch.float32) * (-math.log(10000.0) / d_model))
        pe = torch.zeros(max_len, d_model)
        pe[:, 0::2] = torch.sin(pos * div)
        pe[:, 1::2] = torch.cos(pos * div)[:, : d_model // 2]
        self.register_buffer("pe", pe)
        self.drop = Dropout(dropout)

    def forward(self, x, start_pos: int = 0):
        S = x.shape[-2]
        return self.drop(x + self.pe[start_pos:start_pos + S].to(x.dtype))


class RotaryEmbedding(Module):
    """Rotary position embedding. ``apply(q, k, start_pos)`` rotates ``[B, S, H, D]`` tensors."""

    def __init__(self, dim: int, max_seq_len: int = 2048, theta: float = 10000.0, interleaved: bool = False):
        super().__init__()
        self.dim, self.max_seq_len, self.theta, self.interleaved = dim, max_seq_len, theta, interleaved
        cos, sin = ops.rope_tables(max_seq_len, dim, theta, "cpu")
        self.register_buffer("cos", cos.clone(), persistent=False)
        self.register_buffer("sin", sin.clone(), persistent=False)

    def apply(self, q, k, start_pos: int = 0):
        return (ops.rope(q, self.cos, self.sin, self.interleaved, start_pos),
                ops.rope(k, self.cos, self.sin, self.interleaved, start_pos))

    def forward(self, x, start_pos: int = 0):
        return ops.rope(x, self.cos, self.sin, self.interleaved, start_pos)
