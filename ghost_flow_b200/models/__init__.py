"""Model zoo with the reference's preset names."""
from .configs import BertConfig, GPTConfig, LLaMAConfig, MixtralConfig, T5Config, ViTConfig  # noqa: F401
from .gpt import GPTForCausalLM, GPTForSequenceClassification, GPTModel  # noqa: F401
from .llama import LLaMAForCausalLM, LLaMAModel  # noqa: F401
