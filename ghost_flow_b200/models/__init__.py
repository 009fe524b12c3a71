"""Model zoo with the reference's preset names."""
from .configs import BertConfig, GPTConfig, LLaMAConfig, MixtralConfig, T5Config, ViTConfig  # noqa: F401
from .gpt import GPTForCausalLM, GPTForSequenceClassification, GPTModel  # noqa: F401
from .llama import LLaMAForCausalLM, LLaMAModel  # noqa: F401
from .encoders import (  # noqa: F401
    BertForMaskedLM, BertForSequenceClassification, BertForTokenClassification, BertModel, BertOutput,
    MixtralForCausalLM, PatchEmbedding, T5ForConditionalGeneration, T5Embeddings, T5ForSequenceClassification, T5Model, T5Output,
    VisionTransformer,
)
from .multimodal import (  # noqa: F401
    CLIP, CLIPConfig, CLIPTextConfig, CLIPTextLayer, CLIPVisionConfig, DDPM, BetaSchedule, DiffusionConfig, NeRF, NeRFConfig, NeRFMLP, NoiseScheduler,
    PositionalEncoder, RaySampler, ResidualBlock, UNet, VolumeRenderer,
)
from .geometry import (  # noqa: F401
    ActorCriticAgent, AggregatorType, DQNAgent, FarthestPointSampler, GATLayer, GCNLayer, Graph, GraphSAGELayer, KNNGrouper, Mesh,
    MeshConv, MeshEncoder, MeshPool, MeshUtils, MPNNLayer, PointNet, PointNetBackbone, PointNetConfig, PolicyNetwork,
    Experience, PPOAgent, QNetwork, REINFORCEAgent, ReplayBuffer, SAGEAggregator, STN3d, ValueNetwork,
)
from .vision import (  # noqa: F401
    VGG, BasicBlock, Bottleneck, ChannelsLastEngine, InvertedResidual, MobileNetV2, ResNet, resnet18, resnet34,
    resnet50, resnet101, resnet152, vgg11, vgg16, vgg19,
)
