"""Model configuration dataclasses with the reference's preset names.

LLaMA presets: ghostflow-nn/src/llama.rs:37-138. GPT presets: ghostflow-nn/src/gpt.rs:37-160.
BERT: ghostflow-nn/src/bert.rs:41-86. ViT: ghostflow-nn/src/vision_transformer.rs:38-86.
T5: ghostflow-nn/src/t5.rs:17-127. Mixtral has no preset in the reference; ``MixtralConfig`` combines its
GQA fields (llama.rs:28) with its MoE defaults (ghostflow-nn/src/mixture_of_experts.rs:44-56).
"""
from __future__ import annotations

from dataclasses import dataclass, replace


@dataclass
class LLaMAConfig:
    vocab_size: int = 32000
    hidden_size: int = 4096
    intermediate_size: int = 11008
    num_hidden_layers: int = 32
    num_attention_heads: int = 32
    num_key_value_heads: int = 32
    max_position_embeddings: int = 2048
    rms_norm_eps: float = 1e-6
    rope_theta: float = 10000.0
    rope_interleaved: bool = False
    initializer_range: float = 0.02
    tie_word_embeddings: bool = False

    @property
    def head_dim(self) -> int:
        return self.hidden_size // self.num_attention_heads

    @classmethod
    def llama_7b(cls): return cls()
    @classmethod
    def llama_13b(cls): return cls(hidden_size=5120, intermediate_size=13824, num_hidden_layers=40,
                                   num_attention_heads=40, num_key_value_heads=40)
    @classmethod
    def llama_30b(cls): return cls(hidden_size=6656, intermediate_size=17920, num_hidden_layers=60,
                                   num_attention_heads=52, num_key_value_heads=52)
    @classmethod
    def llama_65b(cls): return cls(hidden_size=8192, intermediate_size=22016, num_hidden_layers=80,
                                   num_attention_heads=64, num_key_value_heads=64)
    @classmethod
    def llama2_7b(cls): return cls(max_position_embeddings=4096)
    @classmethod
    def llama2_13b(cls): return replace(cls.llama_13b(), max_position_embeddings=4096)
    @classmethod
    def llama2_70b(cls): return cls(hidden_size=8192, intermediate_size=28672, num_hidden_layers=80,
                                    num_attention_heads=64, num_key_value_heads=8, max_position_embeddings=4096)
    @classmethod
    def llama_tiny(cls): return cls(vocab_size=1000, hidden_size=128, intermediate_size=512, num_hidden_layers=2,
                                    num_attention_heads=4, num_key_value_heads=4, max_position_embeddings=128)

    def num_parameters(self) -> int:
        d, f, v = self.hidden_size, self.intermediate_size, self.vocab_size
        kv = self.num_key_value_heads * self.head_dim
        per_layer = 2 * d + d * (d + 2 * kv) + d * d + 3 * d * f
        head = 0 if self.tie_word_embeddings else v * d
        return self.num_hidden_layers * per_layer + v * d + d + head


@dataclass
class MixtralConfig(LLaMAConfig):
    intermediate_size: int = 14336
    num_key_value_heads: int = 8
    max_position_embeddings: int = 4096
    num_local_experts: int = 8
    num_experts_per_tok: int = 2
    router_aux_loss_coef: float = 0.01
    capacity_factor: float = 0.0  # 0 = dropless

    @classmethod
    def mixtral_8x7b(cls): return cls()
    @classmethod
    def mixtral_tiny(cls): return cls(vocab_size=1000, hidden_size=128, intermediate_size=256, num_hidden_layers=2,
                                      num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=128,
                                      num_local_experts=4, num_experts_per_tok=2)


@dataclass
class GPTConfig:
    vocab_size: int = 50257
    n_positions: int = 1024
    n_embd: int = 768
    n_layer: int = 12
    n_head: int = 12
    n_inner: int = 3072
    dropout: float = 0.1
    layer_norm_eps: float = 1e-5
    activation: str = "gelu"
    tie_word_embeddings: bool = True
    pre_norm: bool = True
    causal: bool = True
    initializer: str = "normal"   # "normal" (std 0.02) or "xavier_uniform"

    @classmethod
    def gpt2_small(cls): return cls()
    @classmethod
    def gpt2_medium(cls): return cls(n_embd=1024, n_layer=24, n_head=16, n_inner=4096)
    @classmethod
    def gpt2_large(cls): return cls(n_embd=1280, n_layer=36, n_head=20, n_inner=5120)
    @classmethod
    def gpt2_xl(cls): return cls(n_embd=1600, n_layer=48, n_head=25, n_inner=6400)
    @classmethod
    def gpt3_small(cls): return cls(n_positions=2048)
    @classmethod
    def gpt3_medium(cls): return cls(n_positions=2048, n_embd=1024, n_layer=24, n_head=16, n_inner=4096)
    @classmethod
    def gpt3_large(cls): return cls(n_positions=2048, n_embd=1536, n_layer=24, n_head=16, n_inner=6144)
    @classmethod
    def gpt3_xl(cls): return cls(n_positions=2048, n_embd=2048, n_layer=24, n_head=24, n_inner=8192)
    @classmethod
    def gpt_tiny(cls): return cls(vocab_size=1000, n_positions=128, n_embd=128, n_layer=2, n_head=2, n_inner=512)


@dataclass
class BertConfig:
    vocab_size: int = 30522
    hidden_size: int = 768
    num_hidden_layers: int = 12
    num_attention_heads: int = 12
    intermediate_size: int = 3072
    max_position_embeddings: int = 512
    type_vocab_size: int = 2
    hidden_dropout_prob: float = 0.1
    layer_norm_eps: float = 1e-12

    @classmethod
    def bert_base(cls): return cls()
    @classmethod
    def bert_large(cls): return cls(hidden_size=1024, num_hidden_layers=24, num_attention_heads=16,
                                    intermediate_size=4096)
    @classmethod
    def bert_tiny(cls): return cls(vocab_size=1000, hidden_size=128, num_hidden_layers=2, num_attention_heads=2,
                                   intermediate_size=512, max_position_embeddings=128)


@dataclass
class ViTConfig:
    image_size: int = 224
    patch_size: int = 16
    num_channels: int = 3
    hidden_size: int = 768
    num_hidden_layers: int = 12
    num_attention_heads: int = 12
    intermediate_size: int = 3072
    num_classes: int = 1000
    dropout: float = 0.1

    @classmethod
    def vit_base(cls): return cls()
    @classmethod
    def vit_large(cls): return cls(hidden_size=1024, num_hidden_layers=24, num_attention_heads=16,
                                   intermediate_size=4096)
    @classmethod
    def vit_huge(cls): return cls(hidden_size=1280, num_hidden_layers=32, num_attention_heads=16,
                                  intermediate_size=5120)
    @classmethod
    def vit_tiny(cls): return cls(image_size=32, patch_size=8, hidden_size=64, num_hidden_layers=2,
                                  num_attention_heads=2, intermediate_size=128, num_classes=10)

    @property
    def num_patches(self) -> int:
        return (self.image_size // self.patch_size) ** 2


@dataclass
class T5Config:
    vocab_size: int = 32128
    d_model: int = 512
    d_kv: int = 64
    d_ff: int = 2048
    num_layers: int = 6
    num_decoder_layers: int = 6
    num_heads: int = 8
    dropout_rate: float = 0.1
    relative_attention: bool = True
    relative_attention_num_buckets: int = 32

    @classmethod
    def t5_small(cls): return cls()
    @classmethod
    def t5_base(cls): return cls(d_model=768, d_ff=3072, num_layers=12, num_decoder_layers=12, num_heads=12)
    @classmethod
    def t5_large(cls): return cls(d_model=1024, d_ff=4096, num_layers=24, num_decoder_layers=24, num_heads=16)
    @classmethod
    def t5_3b(cls): return cls(d_model=1024, d_kv=128, d_ff=16384, num_layers=24, num_decoder_layers=24,
                               num_heads=32)
    @classmethod
    def t5_11b(cls): return cls(d_model=1024, d_kv=128, d_ff=65536, num_layers=24, num_decoder_layers=24,
                                num_heads=128)
    @classmethod
    def t5_tiny(cls): return cls(vocab_size=1000, d_model=128, d_kv=16, d_ff=512, num_layers=2,
                                 num_decoder_layers=2, num_heads=4)
