"""Neural-network layers, losses and initialisers (see the submodules for reference citations)."""
from . import init  # noqa: F401
from .module import Identity, Module, ModuleDict, ModuleList, Parameter, Sequential  # noqa: F401
from .layers import (  # noqa: F401
    BatchNorm1d, BatchNorm2d, Dropout, Dropout2d, ELU, Embedding, GELU, GroupNorm, InstanceNorm, InstanceNorm2d,
    LayerNorm, LeakyReLU, Linear, LogSoftmax, Mish, ReLU, RMSNorm, SELU, Sigmoid, SiLU, Softmax, Softplus, Swish,
    SwiGLU, SyncBatchNorm, Tanh, TokenPositionEmbedding,
)
from .conv import (  # noqa: F401
    AdaptiveAvgPool2d, AvgPool2d, Conv1d, Conv2d, Conv3d, ConvTranspose2d, Flatten, GlobalAvgPool2d,
    GlobalMaxPool2d, MaxPool2d, TransposeConv2d,
)
from .fused_conv import ConvBNReLU, fold_batch_norm, fuse_conv_bn_relu  # noqa: F401
from .loss import (  # noqa: F401
    BCELoss, BCEWithLogitsLoss, CrossEntropyLoss, FocalLoss, HuberLoss, L1Loss, MSELoss, NLLLoss, SmoothL1Loss,
    binary_cross_entropy, binary_cross_entropy_with_logits, contrastive_loss, cosine_embedding_loss, cross_entropy,
    focal_loss, huber_loss, kl_div_loss, l1_loss, mse_loss, nll_loss, smooth_l1_loss, triplet_margin_loss,
)
from .attention import (  # noqa: F401
    CrossAttention, FlashAttention, FlashAttentionConfig, MultiHeadAttention, scaled_dot_product_attention,
)
from .transformer import RotaryEmbedding as RoPE  # noqa: F401
from .transformer import (  # noqa: F401
    FeedForward, PositionalEncoding, RotaryEmbedding, TransformerDecoder, TransformerDecoderLayer,
    TransformerEncoder, TransformerEncoderLayer,
)
from .rnn import GRU, GRUCell, LSTM, LSTMCell  # noqa: F401
from .mixed_precision import (  # noqa: F401
    AutocastContext, GradScaler, MixedPrecisionConfig, PrecisionMode, autocast, dequantize_fp8_blockwise,
    quantize_fp8_blockwise, to_full_precision, to_half_precision,
)
from .techniques import (  # noqa: F401
    CheckpointConfig, CheckpointedLayer, CheckpointedSequential, CheckpointManager, CheckpointStats,
    CheckpointStrategy, CurriculumConfig, CurriculumLearning, CurriculumStats, CurriculumStrategy,
    DifficultyMetric, DifficultyScorer, DistillationConfig, DistillationMethod, DistillationStats, DynamicQuantization,
    KnowledgeDistillation, LoRAConfig, LoRALinear, PacingFunction, LayerPrefix, PrefixTuning, PrefixTuningConfig, PromptInit, PromptInitStrategy,
    PromptTuning, PromptTuningConfig, PTuningV2, QLoRAConfig, QLoRALinear, QuantType, QuantizationAwareTraining, ScoredSample,
    QuantizationConfig, QuantizationScheme, QuantizedTensor, estimate_memory_savings,
)
from .moe import Expert, MixtureOfExperts, MoEConfig, MoEStats, Router, RoutingStrategy  # noqa: F401
from .ring_attention import RingAttention, RingAttentionConfig, StripedRingAttention  # noqa: F401
from .privacy import (  # noqa: F401
    AdversarialAttack, AdversarialTrainer, AdversarialTrainingConfig, AggregationStrategy, AttackConfig, AttackType,
    DPConfig, DPSGDOptimizer, DifferentialPrivacy, FederatedClient, FederatedServer, LocalDP, PATEEnsemble, PrivacyAccountant,
    RandomizedSmoothing, SecureAggregation,
)
from .inference import (  # noqa: F401
    BatchInference, CudaGraphRunner, FusedOp, InferenceConfig, InferenceOptimizer, InferenceSession, ONNXAttribute, ONNXGraph, ONNXModel,
    ONNXDataType, ONNXNode, ONNXTensor, onnx_to_tensor, tensor_to_onnx, warmup_model,
)
