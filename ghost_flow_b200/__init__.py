"""ghost_flow_b200: a Blackwell-native (sm_100a) deep-learning framework with GhostFlow's capabilities.

``import ghost_flow_b200 as gf`` (or ``import ghost_flow as gf``) gives the reference's Python surface:
``gf.Tensor``, ``gf.randn / rand / zeros / ones``, ``gf.nn``, ``gf.optim`` plus what its documentation
advertises (autograd, losses, ``gf.ml``, ``gf.cuda``) and the distributed trainers in ``gf.parallel``.
"""
__version__ = "0.1.0"

from . import ops  # noqa: F401
from .dtype import DType  # noqa: F401
from .tensor import (  # noqa: F401
    Tensor, enable_grad, get_default_device, manual_seed, no_grad, ones, rand, randn, set_default_device, tensor,
    zeros,
)
from . import nn, optim  # noqa: F401,E402
from . import autograd  # noqa: F401,E402
from .core import (  # noqa: F401,E402
    Cpu, Cuda, Device, GhostError, MemoryLayoutOptimizer, Serializable, Shape, StateDict, Strides, TensorElement,
)


def __getattr__(name):
    # heavier subpackages load on first use
    import importlib

    if name in ("models", "parallel", "io", "data", "ml", "serve", "cuda", "utils"):
        return importlib.import_module(f"{__name__}.{name}")
    raise AttributeError(name)
