"""``ghost_flow``: the reference's package name, served by :mod:`ghost_flow_b200`."""
import sys

import ghost_flow_b200 as _impl
from ghost_flow_b200 import *  # noqa: F401,F403
from ghost_flow_b200 import DType, Tensor, nn, optim, ops, __version__  # noqa: F401


def __getattr__(name):
    return getattr(_impl, name)


for _sub in ("nn", "optim", "ops"):
    sys.modules[f"{__name__}.{_sub}"] = getattr(_impl, _sub)
