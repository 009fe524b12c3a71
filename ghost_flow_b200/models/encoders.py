"""BERT, ViT, T5 and Mixtral model families.

* BERT (ghostflow-nn/src/bert.rs:41-514): ``BertEmbeddings`` (token + position + type, LayerNorm), ``BertPooler``
  (tanh), ``BertModel`` -> ``BertOutput(last_hidden_state, pooler_output)``, ``BertForMaskedLM``,
  ``BertForSequenceClassification``, ``BertForTokenClassification``. The attention mask is honoured (the
  reference ignores it, bert.rs:352-353).
* ViT (ghostflow-nn/src/vision_transformer.rs:38-401): ``PatchEmbedding`` (unfold + Linear), cls token, learned
  positions, pre-LN encoder, LayerNorm, classification head.
* T5 (ghostflow-nn/src/t5.rs:17-528): encoder / decoder with RMS-style LayerNorm, bucketed relative position
  bias (the reference has none) and one shared embedding table (the reference allocates three, t5.rs:287-299).
* Mixtral: LLaMA attention with GQA + a sparse MoE feed-forward of SwiGLU experts (no reference preset;
  ``MixtralConfig`` combines ghostflow-nn/src/llama.rs:28 and mixture_of_experts.rs:44-56).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import NamedTuple

import torch
import torch.nn.functional as F

from .. import ops
from ..nn.attention import scaled_dot_product_attention
from ..nn.layers import Dropout, Embedding, LayerNorm, Linear, RMSNorm
from ..nn.module import Module, ModuleList, Parameter
from ..nn.moe import MixtureOfExperts, MoEConfig
from ..nn.transformer import TransformerEncoderLayer
from .configs import BertConfig, MixtralConfig, T5Config, ViTConfig
from .llama import LLaMAAttention


# =========================================================================== BERT
@dataclass
class BertOutput:
    last_hidden_state: torch.Tensor
    pooler_output: torch.Tensor


class BertEmbeddings(Module):
    def __init__(self, cfg: BertConfig):
        super().__init__()
        self.word = Embedding(cfg.vocab_size, cfg.hidden_size)
        self.position = Embedding(cfg.max_position_embeddings, cfg.hidden_size)
        self.token_type = Embedding(cfg.type_vocab_size, cfg.hidden_size)
        self.norm = LayerNorm(cfg.hidden_size, cfg.layer_norm_eps)
        self.drop = Dropout(cfg.hidden_dropout_prob)

    def forward(self, ids, token_type_ids=None):
        S = ids.shape[1]
        pos = torch.arange(S, device=ids.device)
        tt = token_type_ids if token_type_ids is not None else torch.zeros_like(ids)
        return self.drop(self.norm(self.word(ids) + self.position(pos) + self.token_type(tt)))


class BertPooler(Module):
    def __init__(self, cfg: BertConfig):
        super().__init__()
        self.dense = Linear(cfg.hidden_size, cfg.hidden_size)

    def forward(self, h):
        return torch.tanh(self.dense(h[:, 0]))


class BertModel(Module):
    def __init__(self, cfg: BertConfig):
        super().__init__()
        self.cfg = cfg
        self.embeddings = BertEmbeddings(cfg)
        self.layers = ModuleList([
            TransformerEncoderLayer(cfg.hidden_size, cfg.num_attention_heads, cfg.intermediate_size,
                                    cfg.hidden_dropout_prob, pre_norm=False, eps=cfg.layer_norm_eps)
            for _ in range(cfg.num_hidden_layers)])
        self.pooler = BertPooler(cfg)

    def forward(self, ids, attention_mask=None, token_type_ids=None) -> BertOutput:
        x = self.embeddings(ids, token_type_ids)
        mask = attention_mask[:, None, None, :] if attention_mask is not None else None
        for layer in self.layers:
            x = layer(x, mask)
        return BertOutput(x, self.pooler(x))


class BertForMaskedLM(Module):
    def __init__(self, cfg: BertConfig):
        super().__init__()
        self.bert = BertModel(cfg)
        self.transform = Linear(cfg.hidden_size, cfg.hidden_size)
        self.norm = LayerNorm(cfg.hidden_size, cfg.layer_norm_eps)
        self.decoder = Linear(cfg.hidden_size, cfg.vocab_size)

    def forward(self, ids, attention_mask=None, token_type_ids=None, labels=None):
        h = self.bert(ids, attention_mask, token_type_ids).last_hidden_state
        logits = self.decoder(self.norm(ops.gelu(self.transform(h))))
        if labels is None:
            return logits
        return F.cross_entropy(logits.view(-1, logits.shape[-1]).float(), labels.reshape(-1), ignore_index=-100), logits


class BertForSequenceClassification(Module):
    def __init__(self, cfg: BertConfig, num_labels: int = 2):
        super().__init__()
        self.bert = BertModel(cfg)
        self.drop = Dropout(cfg.hidden_dropout_prob)
        self.classifier = Linear(cfg.hidden_size, num_labels)

    def forward(self, ids, attention_mask=None, token_type_ids=None):
        return self.classifier(self.drop(self.bert(ids, attention_mask, token_type_ids).pooler_output))


class BertForTokenClassification(Module):
    def __init__(self, cfg: BertConfig, num_labels: int = 2):
        super().__init__()
        self.bert = BertModel(cfg)
        self.drop = Dropout(cfg.hidden_dropout_prob)
        self.classifier = Linear(cfg.hidden_size, num_labels)

    def forward(self, ids, attention_mask=None, token_type_ids=None):
        return self.classifier(self.drop(self.bert(ids, attention_mask, token_type_ids).last_hidden_state))


# =========================================================================== ViT
class PatchEmbedding(Module):
    def __init__(self, cfg: ViTConfig):
        super().__init__()
        self.patch = cfg.patch_size
        self.proj = Linear(cfg.num_channels * cfg.patch_size * cfg.patch_size, cfg.hidden_size)

    def forward(self, img):
        p = self.patch
        patches = F.unfold(img, kernel_size=p, stride=p).transpose(1, 2)   # [B, N, C*p*p]
        return self.proj(patches)


class VisionTransformer(Module):
    def __init__(self, cfg: ViTConfig):
        super().__init__()
        self.cfg = cfg
        self.patch_embed = PatchEmbedding(cfg)
        self.cls_token = Parameter(torch.zeros(1, 1, cfg.hidden_size))
        self.pos_embed = Parameter(torch.randn(1, cfg.num_patches + 1, cfg.hidden_size) * 0.02)
        self.drop = Dropout(cfg.dropout)
        self.layers = ModuleList([
            TransformerEncoderLayer(cfg.hidden_size, cfg.num_attention_heads, cfg.intermediate_size, cfg.dropout,
                                    pre_norm=True) for _ in range(cfg.num_hidden_layers)])
        self.norm = LayerNorm(cfg.hidden_size)
        self.head = Linear(cfg.hidden_size, cfg.num_classes)

    def forward_features(self, img):
        x = self.patch_embed(img)
        cls = self.cls_token.to(x.dtype).expand(x.shape[0], -1, -1)
        x = self.drop(torch.cat((cls, x), 1) + self.pos_embed.to(x.dtype))
        for layer in self.layers:
            x = layer(x)
        return self.norm(x)

    def forward(self, img):
        return self.head(self.forward_features(img)[:, 0])


# =========================================================================== T5
class T5LayerNorm(RMSNorm):
    """T5 normalises by the root mean square only (no mean subtraction, no bias)."""


def _relative_bucket(rel, bidirectional: bool, num_buckets: int, max_distance: int = 128):
    ret = torch.zeros_like(rel)
    n = -rel
    if bidirectional:
        num_buckets //= 2
        ret = ret + (n < 0).long() * num_buckets
        n = n.abs()
    else:
        n = n.clamp(min=0)
    max_exact = num_buckets // 2
    is_small = n < max_exact
    large = max_exact + (torch.log(n.float().clamp(min=1) / max_exact) / math.log(max_distance / max_exact)
                         * (num_buckets - max_exact)).long()
    large = large.clamp(max=num_buckets - 1)
    return ret + torch.where(is_small, n, large)


class T5Attention(Module):
    def __init__(self, cfg: T5Config, bidirectional: bool, has_bias: bool):
        super().__init__()
        self.h, self.dk = cfg.num_heads, cfg.d_kv
        inner = cfg.num_heads * cfg.d_kv
        self.q, self.k, self.v = (Linear(cfg.d_model, inner, False) for _ in range(3))
        self.o = Linear(inner, cfg.d_model, False)
        self.bidirectional = bidirectional
        self.num_buckets = cfg.relative_attention_num_buckets
        self.rel_bias = Embedding(self.num_buckets, cfg.num_heads) if (has_bias and cfg.relative_attention) else None

    def bias(self, Sq, Sk, device):
        if self.rel_bias is None:
            return None
        rel = torch.arange(Sk, device=device)[None, :] - torch.arange(Sq, device=device)[:, None]
        b = self.rel_bias(_relative_bucket(rel, self.bidirectional, self.num_buckets))
        return b.permute(2, 0, 1).unsqueeze(0)   # [1, H, Sq, Sk]

    def forward(self, x, kv=None, causal=False, position_bias=None):
        B, Sq, _ = x.shape
        src = x if kv is None else kv
        Sk = src.shape[1]
        q = self.q(x).view(B, Sq, self.h, self.dk).transpose(1, 2)
        k = self.k(src).view(B, Sk, self.h, self.dk).transpose(1, 2)
        v = self.v(src).view(B, Sk, self.h, self.dk).transpose(1, 2)
        s = torch.matmul(q, k.transpose(-1, -2)).float()       # T5 does not scale by sqrt(d)
        if position_bias is None and kv is None:
            position_bias = self.bias(Sq, Sk, x.device)
        if position_bias is not None:
            s = s + position_bias.float()
        if causal:
            s = s.masked_fill(~torch.ones(Sq, Sk, dtype=torch.bool, device=x.device).tril(), float("-inf"))
        o = torch.matmul(torch.softmax(s, -1).to(v.dtype), v).transpose(1, 2).reshape(B, Sq, self.h * self.dk)
        return self.o(o), position_bias


class T5Block(Module):
    def __init__(self, cfg: T5Config, decoder: bool, first: bool):
        super().__init__()
        self.decoder = decoder
        self.ln1 = T5LayerNorm(cfg.d_model)
        self.self_attn = T5Attention(cfg, bidirectional=not decoder, has_bias=first)
        if decoder:
            self.ln_x = T5LayerNorm(cfg.d_model)
            self.cross_attn = T5Attention(cfg, True, False)
        self.ln2 = T5LayerNorm(cfg.d_model)
        self.wi = Linear(cfg.d_model, cfg.d_ff, False)
        self.wo = Linear(cfg.d_ff, cfg.d_model, False)
        self.drop = Dropout(cfg.dropout_rate)

    def forward(self, x, memory=None, position_bias=None):
        a, position_bias = self.self_attn(self.ln1(x), causal=self.decoder, position_bias=position_bias)
        x = x + self.drop(a)
        if self.decoder:
            x = x + self.drop(self.cross_attn(self.ln_x(x), kv=memory)[0])
        return x + self.drop(self.wo(self.drop(torch.relu(self.wi(self.ln2(x)))))), position_bias


class T5Stack(Module):
    def __init__(self, cfg: T5Config, decoder: bool):
        super().__init__()
        n = cfg.num_decoder_layers if decoder else cfg.num_layers
        self.blocks = ModuleList([T5Block(cfg, decoder, i == 0) for i in range(n)])
        self.final_norm = T5LayerNorm(cfg.d_model)
        self.drop = Dropout(cfg.dropout_rate)

    def forward(self, x, memory=None):
        x = self.drop(x)
        bias = None
        for blk in self.blocks:
            x, bias = blk(x, memory, bias)
        return self.drop(self.final_norm(x))


T5Encoder = T5Stack
T5Decoder = T5Stack


class T5Embeddings(Embedding):
    """The token table shared by encoder, decoder and (scaled) output head (ghostflow-nn/src/t5.rs:127-175; there
    the three users hold independent copies, here they share this one module)."""

    def __init__(self, cfg: T5Config):
        super().__init__(cfg.vocab_size, cfg.d_model)
        self.cfg = cfg

    def forward(self, input_ids):
        if input_ids.dim() != 2:
            raise ValueError(f"expected 2-D input_ids, got {input_ids.dim()}-D")
        return super().forward(input_ids)


class T5Model(Module):
    def __init__(self, cfg: T5Config):
        super().__init__()
        self.cfg = cfg
        self.shared = T5Embeddings(cfg)
        self.encoder = T5Stack(cfg, False)
        self.decoder = T5Stack(cfg, True)

    def forward(self, input_ids, decoder_input_ids):
        mem = self.encoder(self.shared(input_ids))
        return T5Output(self.decoder(self.shared(decoder_input_ids), mem), mem)


class T5Output(NamedTuple):
    """Result of the encoder-decoder stack (ghostflow-nn/src/t5.rs:321-328); unpacks as ``(decoder, encoder)``."""
    last_hidden_state: torch.Tensor
    encoder_last_hidden_state: torch.Tensor


class T5ForConditionalGeneration(Module):
    def __init__(self, cfg: T5Config):
        super().__init__()
        self.cfg = cfg
        self.t5 = T5Model(cfg)
        self.lm_head = Linear(cfg.d_model, cfg.vocab_size, False)

    def forward(self, input_ids, decoder_input_ids, labels=None):
        h, _ = self.t5(input_ids, decoder_input_ids)
        logits = self.lm_head(h * (self.cfg.d_model ** -0.5))
        if labels is None:
            return logits
        return F.cross_entropy(logits.view(-1, logits.shape[-1]).float(), labels.reshape(-1), ignore_index=-100), logits

    @torch.no_grad()
    def generate(self, input_ids, max_new_tokens: int = 20, start_token: int = 0, eos_token: int | None = 1):
        mem = self.t5.encoder(self.t5.shared(input_ids))
        out = torch.full((input_ids.shape[0], 1), start_token, dtype=torch.long, device=input_ids.device)
        for _ in range(max_new_tokens):
            h = self.t5.decoder(self.t5.shared(out), mem)
            nxt = self.lm_head(h[:, -1:] * (self.cfg.d_model ** -0.5)).argmax(-1)
            out = torch.cat((out, nxt), 1)
            if eos_token is not None and bool((nxt == eos_token).all()):
                break
        return out


class T5ForSequenceClassification(Module):
    def __init__(self, cfg: T5Config, num_labels: int = 2):
        super().__init__()
        self.shared = Embedding(cfg.vocab_size, cfg.d_model)
        self.encoder = T5Stack(cfg, False)
        self.classifier = Linear(cfg.d_model, num_labels)

    def forward(self, input_ids):
        return self.classifier(self.encoder(self.shared(input_ids)).mean(1))


# =========================================================================== Mixtral
class MixtralDecoderLayer(Module):
    def __init__(self, cfg: MixtralConfig, device=None, dtype=None):
        super().__init__()
        self.attn_norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, device, dtype)
        self.attn = LLaMAAttention(cfg, device, dtype)
        self.ffn_norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, device, dtype)
        self.moe = MixtureOfExperts(MoEConfig(cfg.num_local_experts, cfg.num_experts_per_tok, cfg.hidden_size,
                                              cfg.intermediate_size, aux_loss_weight=cfg.router_aux_loss_coef,
                                              expert_type="swiglu"), device, dtype)

    def forward(self, x, cos, sin):
        x = self.attn(self.attn_norm(x), cos, sin, residual=x)
        return x + self.moe(self.ffn_norm(x))


class MixtralForCausalLM(Module):
    def __init__(self, cfg: MixtralConfig, device=None, dtype=None):
        super().__init__()
        self.cfg = cfg
        self.embed_tokens = Embedding(cfg.vocab_size, cfg.hidden_size, device=device, dtype=dtype)
        self.layers = ModuleList([MixtralDecoderLayer(cfg, device, dtype) for _ in range(cfg.num_hidden_layers)])
        self.norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, device, dtype)
        self.lm_head = Linear(cfg.hidden_size, cfg.vocab_size, False, device, dtype)
        with torch.no_grad():
            for n, p in self.named_parameters():
                if n.endswith("norm.weight"):
                    p.fill_(1.0)
                else:
                    p.normal_(0.0, cfg.initializer_range)

    def forward(self, ids, labels=None):
        S = ids.shape[1]
        cos, sin = ops.rope_tables(max(S, self.cfg.max_position_embeddings), self.cfg.head_dim, self.cfg.rope_theta,
                                   ids.device)
        x = self.embed_tokens(ids)
        for layer in self.layers:
            x = layer(x, cos, sin)
        logits = self.lm_head(self.norm(x))
        if labels is None:
            return logits
        loss = ops.cross_entropy(logits.view(-1, logits.shape[-1]), labels.reshape(-1))
        aux = sum(layer.moe.get_aux_loss() for layer in self.layers)
        return loss + aux.to(loss.dtype), logits

    def aux_loss(self):
        return sum(layer.moe.get_aux_loss() for layer in self.layers)
