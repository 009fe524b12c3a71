"""Training techniques with the reference's class names: gradient checkpointing, LoRA / QLoRA, quantization,
knowledge distillation, prompt / prefix tuning, curriculum learning.

* Gradient checkpointing (ghostflow-nn/src/gradient_checkpointing.rs:14-255): the reference only counts bytes
  and its "backward" returns the gradient unchanged (:187-198); here activations really are dropped and
  recomputed in backward.
* LoRA (ghostflow-nn/src/lora.rs:14-285): ``merge_weights`` really folds ``B A * alpha / r`` into the base
  weight (the reference only flips a flag, :132-156); QLoRA stores NF4 codes with per-block absmax.
* Quantization (ghostflow-nn/src/quantization.rs:77-240): INT8 per-tensor / per-channel, symmetric or
  asymmetric, fake-quant for QAT, dynamic quantization.
* Distillation (knowledge_distillation.rs:15-150), prompt tuning (prompt_tuning.rs:14-400), curriculum
  learning (curriculum_learning.rs:14-380).
"""
from __future__ import annotations

import enum
import math
from dataclasses import dataclass, field

import torch
import torch.nn.functional as F
from torch.utils.checkpoint import checkpoint as _torch_checkpoint

from .layers import Linear
from .module import Module, ModuleList, Parameter


# =========================================================================== gradient checkpointing
class CheckpointStrategy(enum.Enum):
    EveryN = "every_n"
    Selective = "selective"
    All = "all"
    Nothing = "none"


@dataclass
class CheckpointConfig:
    strategy: CheckpointStrategy = CheckpointStrategy.EveryN
    every_n: int = 2
    selected_layers: tuple = ()
    enabled: bool = True


@dataclass
class CheckpointStats:
    num_checkpoints: int = 0
    num_recomputations: int = 0
    memory_saved_bytes: int = 0


class CheckpointManager:
    def __init__(self, config: CheckpointConfig | None = None):
        self.config = config or CheckpointConfig()
        self.stats = CheckpointStats()

    def should_checkpoint(self, layer_idx: int) -> bool:
        c = self.config
        if not c.enabled or c.strategy == CheckpointStrategy.Nothing:
            return False
        if c.strategy == CheckpointStrategy.All:
            return True
        if c.strategy == CheckpointStrategy.EveryN:
            return layer_idx % max(1, c.every_n) == 0
        return layer_idx in c.selected_layers

    def run(self, layer_idx: int, fn, *args):
        if self.should_checkpoint(layer_idx) and torch.is_grad_enabled() and any(
                isinstance(a, torch.Tensor) and a.requires_grad for a in args):
            self.stats.num_checkpoints += 1
            self.stats.memory_saved_bytes += sum(a.numel() * a.element_size() for a in args
                                                 if isinstance(a, torch.Tensor))

            calls = [0]

            def counted(*a):
                calls[0] += 1
                if calls[0] > 1:   # the first call is the forward pass, later ones are recomputations
                    self.stats.num_recomputations += 1
                return fn(*a)

            return _torch_checkpoint(counted, *args, use_reentrant=False)
        return fn(*args)

    def get_stats(self):
        return self.stats


class CheckpointedLayer(Module):
    def __init__(self, layer, manager: CheckpointManager | None = None, index: int = 0):
        super().__init__()
        self.layer = layer
        self.manager = manager or CheckpointManager(CheckpointConfig(CheckpointStrategy.All))
        self.index = index

    def forward(self, *args):
        return self.manager.run(self.index, self.layer, *args)


class CheckpointedSequential(Module):
    def __init__(self, layers, config: CheckpointConfig | None = None):
        super().__init__()
        self.layers = ModuleList(layers)
        self.manager = CheckpointManager(config)

    def forward(self, x):
        for i, layer in enumerate(self.layers):
            x = self.manager.run(i, layer, x)
        return x


def estimate_memory_savings(num_layers: int, config: CheckpointConfig) -> float:
    """Fraction of activation memory saved (ghostflow-nn/src/gradient_checkpointing.rs estimate)."""
    m = CheckpointManager(config)
    kept = sum(1 for i in range(num_layers) if not m.should_checkpoint(i))
    return 1.0 - kept / max(1, num_layers)


# =========================================================================== LoRA / QLoRA
@dataclass
class LoRAConfig:
    rank: int = 8
    alpha: float = 16.0
    dropout: float = 0.0
    merge_weights: bool = False

    @property
    def scaling(self):
        return self.alpha / self.rank


class LoRALinear(Module):
    def __init__(self, in_features, out_features, config: LoRAConfig | None = None, bias: bool = True):
        super().__init__()
        self.config = config or LoRAConfig()
        self.base = Linear(in_features, out_features, bias)
        for p in self.base.parameters():
            p.requires_grad_(False)
        r = self.config.rank
        self.lora_a = Parameter(torch.randn(r, in_features) * (1.0 / math.sqrt(in_features)))
        self.lora_b = Parameter(torch.zeros(out_features, r))
        self.merged = False

    def forward(self, x):
        y = self.base(x)
        if self.merged:
            return y
        h = F.dropout(x, self.config.dropout, self.training)
        return y + (h @ self.lora_a.t().to(x.dtype)) @ self.lora_b.t().to(x.dtype) * self.config.scaling

    @torch.no_grad()
    def merge_weights(self):
        if not self.merged:
            self.base.weight += (self.lora_b @ self.lora_a).to(self.base.weight.dtype) * self.config.scaling
            self.merged = True

    @torch.no_grad()
    def unmerge_weights(self):
        if self.merged:
            self.base.weight -= (self.lora_b @ self.lora_a).to(self.base.weight.dtype) * self.config.scaling
            self.merged = False

    def lora_parameters(self):
        return [self.lora_a, self.lora_b]


_NF4 = torch.tensor([-1.0, -0.6961928009986877, -0.5250730514526367, -0.39491748809814453, -0.28444138169288635,
                     -0.18477343022823334, -0.09105003625154495, 0.0, 0.07958029955625534, 0.16093020141124725,
                     0.24611230194568634, 0.33791524171829224, 0.44070982933044434, 0.5626170039176941,
                     0.7229568362236023, 1.0])


# the sixteen e2m1 values (sign, 2 exponent bits, 1 mantissa bit) scaled to [-1, 1]
_FP4 = torch.tensor(sorted({s * v / 6.0 for s in (-1.0, 1.0) for v in (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)})
                    + [1.0])[:16]


class QuantType(enum.Enum):
    """Storage format of a frozen QLoRA base weight (ghostflow-nn/src/lora.rs:187-196): a code book of values in
    [-1, 1] indexed by the stored code, times the per-block absmax. NF4 = the sixteen normal-float quantiles,
    FP4 = the e2m1 values, INT8 = 255 evenly spaced levels (symmetric int8)."""
    NF4 = "nf4"
    FP4 = "fp4"
    INT8 = "int8"

    def code_book(self) -> torch.Tensor:
        if self is QuantType.NF4:
            return _NF4
        if self is QuantType.FP4:
            return _FP4
        return torch.arange(-127, 128, dtype=torch.float32) / 127.0


@dataclass
class QLoRAConfig(LoRAConfig):
    bits: int = 4
    double_quant: bool = True
    quant_type: str = "nf4"
    block_size: int = 64


class QLoRALinear(Module):
    """LoRA over a frozen 4-bit NF4 base weight (per-block absmax; absmax itself stored in 8 bits when
    ``double_quant``)."""

    def __init__(self, in_features, out_features, config: QLoRAConfig | None = None):
        super().__init__()
        self.config = config or QLoRAConfig()
        self.in_features, self.out_features = in_features, out_features
        w = torch.empty(out_features, in_features)
        from . import init

        init.kaiming_uniform(w)
        self._quantize(w)
        r = self.config.rank
        self.lora_a = Parameter(torch.randn(r, in_features) * (1.0 / math.sqrt(in_features)))
        self.lora_b = Parameter(torch.zeros(out_features, r))

    def _quantize(self, w):
        bs = self.config.block_size
        flat = w.reshape(-1)
        pad = (-flat.numel()) % bs
        flat = F.pad(flat, (0, pad))
        blocks = flat.view(-1, bs)
        absmax = blocks.abs().amax(1).clamp(min=1e-12)
        qt = self.config.quant_type
        self.quant_type = qt if isinstance(qt, QuantType) else QuantType(str(qt).lower())
        book = self.quant_type.code_book()
        norm = blocks / absmax[:, None]
        # nearest code-book entry, in chunks (an int8 book has 255 entries)
        codes = torch.cat([c.unsqueeze(-1).sub(book).abs().argmin(-1) for c in norm.split(4096)]).to(torch.uint8)
        self.register_buffer("codes", codes)
        if self.config.double_quant:
            s = absmax.max() / 255.0
            self.register_buffer("absmax_q", torch.round(absmax / s).to(torch.uint8))
            self.register_buffer("absmax_scale", s.reshape(1))
        else:
            self.register_buffer("absmax", absmax)
        self._pad = pad

    def dequantize(self):
        absmax = self.absmax_q.float() * self.absmax_scale if self.config.double_quant else self.absmax
        w = self.quant_type.code_book().to(self.codes.device)[self.codes.long()] * absmax[:, None]
        w = w.reshape(-1)
        if self._pad:
            w = w[:-self._pad]
        return w.view(self.out_features, self.in_features)

    def forward(self, x):
        w = self.dequantize().to(x.dtype)
        return x @ w.t() + (x @ self.lora_a.t().to(x.dtype)) @ self.lora_b.t().to(x.dtype) * self.config.scaling


# =========================================================================== quantization
class QuantizationScheme(enum.Enum):
    INT8 = "int8"
    FP16 = "fp16"
    Dynamic = "dynamic"


@dataclass
class QuantizationConfig:
    scheme: QuantizationScheme = QuantizationScheme.INT8
    per_channel: bool = False
    symmetric: bool = True
    channel_dim: int = 0


class QuantizedTensor:
    """INT8 (or fp16) storage with scale / zero-point, per tensor or per channel."""

    def __init__(self, data, scale, zero_point, shape, config: QuantizationConfig):
        self.data, self.scale, self.zero_point, self.shape, self.config = data, scale, zero_point, shape, config

    @classmethod
    def from_tensor(cls, t: torch.Tensor, config: QuantizationConfig | None = None):
        config = config or QuantizationConfig()
        t = getattr(t, "data", t) if not isinstance(t, torch.Tensor) else t
        if config.scheme == QuantizationScheme.FP16:
            return cls(t.to(torch.float16), None, None, tuple(t.shape), config)
        x = t.float()
        if config.per_channel:
            dims = [d for d in range(x.dim()) if d != config.channel_dim]
            mn, mx = x.amin(dims, keepdim=True), x.amax(dims, keepdim=True)
        else:
            mn, mx = x.min(), x.max()
        if config.symmetric:
            scale = (torch.maximum(mn.abs(), mx.abs()) / 127.0).clamp(min=1e-12)
            zp = torch.zeros_like(scale)
            q = torch.round(x / scale).clamp(-127, 127)
        else:
            scale = ((mx - mn) / 255.0).clamp(min=1e-12)
            zp = torch.round(-mn / scale) - 128
            q = (torch.round(x / scale) + zp).clamp(-128, 127)
        return cls(q.to(torch.int8), scale, zp, tuple(t.shape), config)

    def dequantize(self) -> torch.Tensor:
        if self.config.scheme == QuantizationScheme.FP16:
            return self.data.float()
        return (self.data.float() - self.zero_point) * self.scale

    def compression_ratio(self) -> float:
        return 4.0 / self.data.element_size()


class QuantizationAwareTraining:
    """Fake quantisation with a straight-through gradient."""

    def __init__(self, config: QuantizationConfig | None = None):
        self.config = config or QuantizationConfig()

    def fake_quantize(self, t: torch.Tensor) -> torch.Tensor:
        x = getattr(t, "data", t) if not isinstance(t, torch.Tensor) else t
        dq = QuantizedTensor.from_tensor(x.detach(), self.config).dequantize().to(x.dtype)
        return x + (dq - x).detach()


class DynamicQuantization:
    """Quantises activations on the fly per call and runs the matmul on dequantised values."""

    def __init__(self, config: QuantizationConfig | None = None):
        self.config = config or QuantizationConfig(QuantizationScheme.Dynamic)

    def quantize(self, t):
        return QuantizedTensor.from_tensor(t, QuantizationConfig(QuantizationScheme.INT8, False, True))

    def linear(self, x, qweight: QuantizedTensor, bias=None):
        xq = self.quantize(x)
        return F.linear(xq.dequantize(), qweight.dequantize(), bias)


# =========================================================================== knowledge distillation
class DistillationMethod(enum.Enum):
    Standard = "standard"
    Feature = "feature"
    Attention = "attention"
    FitNet = "fitnet"
    Progressive = "progressive"


@dataclass
class DistillationConfig:
    temperature: float = 4.0
    alpha: float = 0.7
    beta: float = 0.3
    method: DistillationMethod = DistillationMethod.Standard
    feature_layers: tuple = ()

    @classmethod
    def standard(cls, temperature, alpha): return cls(temperature, alpha, 1.0 - alpha)
    @classmethod
    def feature_based(cls, temperature, layers): return cls(temperature, method=DistillationMethod.Feature,
                                                            feature_layers=tuple(layers))
    @classmethod
    def attention_transfer(cls, temperature): return cls(temperature, method=DistillationMethod.Attention)


@dataclass
class DistillationStats:
    steps: int = 0
    last_soft_loss: float = 0.0
    last_hard_loss: float = 0.0


class KnowledgeDistillation:
    def __init__(self, config: DistillationConfig | None = None):
        self.config = config or DistillationConfig()
        self.stats = DistillationStats()

    def compute_loss(self, student_logits, teacher_logits, targets, student_features=None, teacher_features=None):
        """``alpha * T^2 * KL(teacher_T || student_T) + beta * CE(student, targets)`` (+ feature / attention terms)."""
        c = self.config
        T = c.temperature
        ls = F.log_softmax(student_logits.float() / T, -1)
        pt = F.softmax(teacher_logits.float() / T, -1)
        soft = F.kl_div(ls, pt, reduction="batchmean") * T * T
        hard = F.cross_entropy(student_logits.float(), targets.long())
        loss = c.alpha * soft + c.beta * hard
        if c.method in (DistillationMethod.Feature, DistillationMethod.FitNet) and student_features is not None:
            loss = loss + sum(F.mse_loss(s.float(), t.float()) for s, t in zip(student_features, teacher_features))
        if c.method == DistillationMethod.Attention and student_features is not None:
            def amap(f):
                a = f.float().pow(2).mean(1).flatten(1)
                return F.normalize(a, dim=1)
            loss = loss + sum((amap(s) - amap(t)).pow(2).mean() for s, t in zip(student_features, teacher_features))
        self.stats.steps += 1
        self.stats.last_soft_loss, self.stats.last_hard_loss = float(soft), float(hard)
        return loss

    def get_stats(self):
        return self.stats


# =========================================================================== prompt / prefix tuning
class PromptInit(enum.Enum):
    Random = "random"
    Vocab = "vocab"
    Text = "text"


PromptInitStrategy = PromptInit     # the reference's name (ghostflow-nn/src/prompt_tuning.rs:27-36)


@dataclass
class PromptTuningConfig:
    num_virtual_tokens: int = 20
    d_model: int = 768
    init: PromptInit = PromptInit.Random
    reparameterization: bool = False
    hidden_size: int = 512

    @classmethod
    def short(cls, d_model=768): return cls(10, d_model)
    @classmethod
    def medium(cls, d_model=768): return cls(30, d_model)
    @classmethod
    def long(cls, d_model=768): return cls(80, d_model)

    def with_reparameterization(self, hidden):
        self.reparameterization, self.hidden_size = True, hidden
        return self


class PromptTuning(Module):
    def __init__(self, config: PromptTuningConfig | None = None, vocab_embeddings: torch.Tensor | None = None):
        super().__init__()
        self.config = c = config or PromptTuningConfig()
        if c.init == PromptInit.Vocab and vocab_embeddings is not None:
            idx = torch.randint(0, vocab_embeddings.shape[0], (c.num_virtual_tokens,))
            init = vocab_embeddings[idx].detach().clone().float()
        else:
            init = torch.randn(c.num_virtual_tokens, c.d_model) * 0.02
        self.prompt = Parameter(init)
        if c.reparameterization:
            self.mlp = torch.nn.Sequential(torch.nn.Linear(c.d_model, c.hidden_size), torch.nn.Tanh(),
                                           torch.nn.Linear(c.hidden_size, c.d_model))

    def get_prompt_embeddings(self):
        return self.prompt + self.mlp(self.prompt) if self.config.reparameterization else self.prompt

    def prepend_prompts(self, embeddings):
        """embeddings ``[B, S, D]`` -> ``[B, P + S, D]``."""
        p = self.get_prompt_embeddings().to(embeddings.dtype).unsqueeze(0).expand(embeddings.shape[0], -1, -1)
        return torch.cat((p, embeddings), dim=1)

    forward = prepend_prompts


@dataclass
class PrefixTuningConfig:
    num_prefix_tokens: int = 10
    num_layers: int = 12
    d_model: int = 768
    num_heads: int = 12
    prefix_kv: bool = True

    @classmethod
    def small(cls): return cls(5)
    @classmethod
    def large(cls): return cls(20)


@dataclass
class LayerPrefix:
    """Key and value prefix of one layer (ghostflow-nn/src/prompt_tuning.rs:252-259)."""
    prefix_key: torch.Tensor
    prefix_value: torch.Tensor


class PrefixTuning(Module):
    def __init__(self, config: PrefixTuningConfig | None = None):
        super().__init__()
        self.config = c = config or PrefixTuningConfig()
        self.prefix = Parameter(torch.randn(c.num_layers, 2, c.num_prefix_tokens, c.d_model) * 0.02)

    def layer_prefix(self, layer: int) -> "LayerPrefix":
        """The pair of :meth:`get_layer_prefix` as the reference's record type."""
        return LayerPrefix(*self.get_layer_prefix(layer))

    def get_layer_prefix(self, layer: int):
        """(key_prefix, value_prefix), each ``[P, H, D/H]``."""
        c = self.config
        k, v = self.prefix[layer, 0], self.prefix[layer, 1]
        hd = c.d_model // c.num_heads
        return k.view(c.num_prefix_tokens, c.num_heads, hd), v.view(c.num_prefix_tokens, c.num_heads, hd)

    def prepend_to_kv(self, layer: int, k, v):
        """k, v ``[B, S, H, D]`` -> ``[B, P + S, H, D]``."""
        pk, pv = self.get_layer_prefix(layer)
        B = k.shape[0]
        return (torch.cat((pk.to(k.dtype).unsqueeze(0).expand(B, -1, -1, -1), k), 1),
                torch.cat((pv.to(v.dtype).unsqueeze(0).expand(B, -1, -1, -1), v), 1))


class PTuningV2(PrefixTuning):
    """Deep prompt tuning: a prefix at every layer produced by a small re-parameterisation MLP."""

    def __init__(self, config: PrefixTuningConfig | None = None, hidden: int = 512):
        super().__init__(config)
        c = self.config
        self.encoder = torch.nn.Sequential(torch.nn.Linear(c.d_model, hidden), torch.nn.Tanh(),
                                           torch.nn.Linear(hidden, c.d_model))

    def get_layer_prefix(self, layer: int):
        c = self.config
        kv = self.encoder(self.prefix[layer])
        hd = c.d_model // c.num_heads
        return (kv[0].view(c.num_prefix_tokens, c.num_heads, hd), kv[1].view(c.num_prefix_tokens, c.num_heads, hd))


# =========================================================================== curriculum learning
class CurriculumStrategy(enum.Enum):
    Fixed = "fixed"
    SelfPaced = "self_paced"
    TeacherStudent = "teacher_student"
    CompetenceBased = "competence_based"
    AntiCurriculum = "anti_curriculum"


class DifficultyMetric(enum.Enum):
    """How a sample's difficulty is scored (ghostflow-nn/src/curriculum_learning.rs:27-38)."""
    Loss = "loss"
    Confidence = "confidence"      # difficulty = 1 - confidence of the prediction
    Complexity = "complexity"      # length / feature count handed in by the caller
    Custom = "custom"              # user function


class PacingFunction(enum.Enum):
    Linear = "linear"
    Exponential = "exponential"
    Step = "step"
    Root = "root"


@dataclass
class CurriculumConfig:
    strategy: CurriculumStrategy = CurriculumStrategy.Fixed
    metric: str = "loss"                      # or a DifficultyMetric (``difficulty_metric`` is the reference's name)
    initial_threshold: float = 0.3
    final_threshold: float = 1.0
    warmup_epochs: int = 10
    pacing: PacingFunction = PacingFunction.Linear
    min_samples_per_batch: int = 8

    @classmethod
    def self_paced(cls, warmup): return cls(CurriculumStrategy.SelfPaced, warmup_epochs=warmup)
    @classmethod
    def competence_based(cls, warmup): return cls(CurriculumStrategy.CompetenceBased, warmup_epochs=warmup,
                                                  pacing=PacingFunction.Root)
    @classmethod
    def anti_curriculum(cls): return cls(CurriculumStrategy.AntiCurriculum, initial_threshold=1.0,
                                         final_threshold=0.0)


CurriculumConfig.difficulty_metric = property(
    lambda self: DifficultyMetric(self.metric.value if isinstance(self.metric, DifficultyMetric) else self.metric))


@dataclass
class CurriculumStats:
    epoch: int = 0
    threshold: float = 0.0
    num_selected: int = 0
    num_total: int = 0


class DifficultyScorer:
    """Scores samples in [0, 1]: normalised loss, sequence length or a user function."""

    def __init__(self, metric="loss", fn=None):
        self.metric = metric.value if isinstance(metric, DifficultyMetric) else metric
        self.fn = fn
        if self.metric == "custom" and fn is None:
            raise ValueError("DifficultyMetric.Custom needs a scoring function")

    def score(self, values):
        if self.fn is not None:
            v = torch.as_tensor([self.fn(x) for x in values], dtype=torch.float32)
        else:
            v = torch.as_tensor(values, dtype=torch.float32)
        if self.metric == "confidence":
            v = 1.0 - v                                   # a confident prediction is an easy sample
        lo, hi = v.min(), v.max()
        return (v - lo) / (hi - lo).clamp(min=1e-12)


@dataclass
class ScoredSample:
    """A sample with its difficulty (ghostflow-nn/src/curriculum_learning.rs:116-127)."""
    index: int
    difficulty: float                 # 0 = easy, 1 = hard
    loss: float | None = None
    metadata: dict = field(default_factory=dict)


class CurriculumLearning:
    def __init__(self, config: CurriculumConfig | None = None):
        self.config = config or CurriculumConfig()
        self.epoch = 0
        self.difficulties = None
        self.threshold = self.config.initial_threshold

    def initialize_samples(self, difficulties):
        self.difficulties = DifficultyScorer().score(difficulties)

    def _progress(self) -> float:
        c = self.config
        t = min(1.0, self.epoch / max(1, c.warmup_epochs))
        if c.pacing == PacingFunction.Exponential:
            return (math.exp(3 * t) - 1) / (math.exp(3) - 1)
        if c.pacing == PacingFunction.Step:
            return math.floor(t * 4) / 4
        if c.pacing == PacingFunction.Root:
            return math.sqrt(t)
        return t

    def update_threshold(self) -> float:
        c = self.config
        self.threshold = c.initial_threshold + (c.final_threshold - c.initial_threshold) * self._progress()
        return self.threshold

    def select_samples(self):
        """Indices of the samples admitted at the current threshold (hardest first for anti-curriculum)."""
        assert self.difficulties is not None, "call initialize_samples first"
        d = self.difficulties
        if self.config.strategy == CurriculumStrategy.AntiCurriculum:
            idx = torch.nonzero(d >= self.threshold).flatten()
            order = torch.argsort(d, descending=True)
        else:
            idx = torch.nonzero(d <= self.threshold).flatten()
            order = torch.argsort(d)
        if idx.numel() < self.config.min_samples_per_batch:
            idx = order[: self.config.min_samples_per_batch]
        return idx

    def update_sample_losses(self, indices, losses):
        """Self-paced / competence-based: difficulty follows the current per-sample loss."""
        if self.config.strategy in (CurriculumStrategy.SelfPaced, CurriculumStrategy.CompetenceBased,
                                    CurriculumStrategy.TeacherStudent):
            l = torch.as_tensor(losses, dtype=torch.float32)
            self.difficulties[torch.as_tensor(indices)] = (l / l.max().clamp(min=1e-12)).clamp(0, 1)

    def scored_samples(self, losses=None) -> list:
        """Every sample as a :class:`ScoredSample`, easiest first (``losses``: optional per-sample losses)."""
        assert self.difficulties is not None, "call initialize_samples first"
        order = torch.argsort(self.difficulties)
        return [ScoredSample(int(i), float(self.difficulties[i]), None if losses is None else float(losses[int(i)]))
                for i in order]

    def next_epoch(self):
        self.epoch += 1
        return self.update_threshold()

    def get_stats(self):
        n = 0 if self.difficulties is None else int(self.difficulties.numel())
        sel = 0 if self.difficulties is None else int(self.select_samples().numel())
        return CurriculumStats(self.epoch, self.threshold, sel, n)
