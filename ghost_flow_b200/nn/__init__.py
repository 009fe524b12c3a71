"""Neural-network layers, losses and initialisers (see the submodules for reference citations)."""
from . import init  # noqa: F401
from .module import Identity, Module, ModuleDict, ModuleList, Parameter, Sequential  # noqa: F401
from .layers import (  # noqa: F401
    BatchNorm1d, BatchNorm2d, Dropout, Dropout2d, ELU, Embedding, GELU, GroupNorm, InstanceNorm, InstanceNorm2d,
    LayerNorm, LeakyReLU, Linear, LogSoftmax, Mish, ReLU, RMSNorm, SELU, Sigmoid, SiLU, Softmax, Softplus, Swish,
    SwiGLU, Tanh, TokenPositionEmbedding,
)
from .conv import (  # noqa: F401
    AdaptiveAvgPool2d, AvgPool2d, Conv1d, Conv2d, Conv3d, ConvTranspose2d, Flatten, GlobalAvgPool2d,
    GlobalMaxPool2d, MaxPool2d, TransposeConv2d,
)
from .loss import (  # noqa: F401
    BCELoss, BCEWithLogitsLoss, CrossEntropyLoss, FocalLoss, HuberLoss, L1Loss, MSELoss, NLLLoss, SmoothL1Loss,
    binary_cross_entropy, binary_cross_entropy_with_logits, contrastive_loss, cosine_embedding_loss, cross_entropy,
    focal_loss, huber_loss, kl_div_loss, l1_loss, mse_loss, nll_loss, smooth_l1_loss, triplet_margin_loss,
)
from .attention import (  # noqa: F401
    CrossAttention, FlashAttention, FlashAttentionConfig, MultiHeadAttention, scaled_dot_product_attention,
)
from .transformer import (  # noqa: F401
    FeedForward, PositionalEncoding, RotaryEmbedding, TransformerDecoder, TransformerDecoderLayer,
    TransformerEncoder, TransformerEncoderLayer,
)
from .rnn import GRU, GRUCell, LSTM, LSTMCell  # noqa: F401
