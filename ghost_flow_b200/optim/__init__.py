"""Optimizers and learning-rate schedulers."""
from .optimizers import SGD, Adam, AdamW, Optimizer, ParamGroup, clip_grad_norm_  # noqa: F401
from .extra import Adadelta, AdaGrad, Adagrad, RMSprop  # noqa: F401
from .schedulers import (  # noqa: F401
    CosineAnnealingLR, ExponentialLR, LinearWarmup, LRScheduler, ReduceLROnPlateau, StepLR, WarmupCosine,
)
