"""``Module`` / ``Sequential``: the reference's trait surface (ghostflow-nn/src/module.rs:6-87:
``forward, parameters, num_parameters, train, eval, is_training``, ``Sequential::new().add_layer()``)
on top of ``torch.nn.Module``, which adds what the reference lacks: names, ``state_dict``,
``zero_grad`` and ``to(device)``. Modules accept and return :class:`ghost_flow_b200.Tensor` or raw
``torch.Tensor`` (whichever they were given).
"""
from __future__ import annotations

import torch

from ..tensor import Tensor

Parameter = torch.nn.Parameter
ModuleList = torch.nn.ModuleList
ModuleDict = torch.nn.ModuleDict
Identity = torch.nn.Identity


def _unwrap_args(args, kwargs):
    wrapped = False

    def u(x):
        nonlocal wrapped
        if isinstance(x, Tensor):
            wrapped = True
            return x.data
        if isinstance(x, (list, tuple)):
            return type(x)(u(y) for y in x)
        return x

    return tuple(u(a) for a in args), {k: u(v) for k, v in kwargs.items()}, wrapped


def _wrap_out(out):
    if isinstance(out, torch.Tensor):
        return Tensor(out)
    if isinstance(out, tuple):
        return tuple(_wrap_out(o) for o in out)
    if isinstance(out, list):
        return [_wrap_out(o) for o in out]
    return out


class Module(torch.nn.Module):
    """Base class of every layer and model."""

    _profile_hook = None  # set by ghost_flow_b200.utils.profiler when profiling of modules is enabled

    def __call__(self, *args, **kwargs):
        a, k, wrapped = _unwrap_args(args, kwargs)
        hook = Module._profile_hook
        if hook is not None:
            with hook(type(self).__name__):
                out = super().__call__(*a, **k)
        else:
            out = super().__call__(*a, **k)
        return _wrap_out(out) if wrapped else out

    @classmethod
    def new(cls, *args, **kwargs):
        """``Linear.new(10, 5)``: the reference's constructor spelling (``Linear::new``), same as ``Linear(10, 5)``."""
        return cls(*args, **kwargs)

    def parameters_list(self):
        return list(self.parameters())

    def num_parameters(self) -> int:
        return sum(p.numel() for p in self.parameters())

    def is_training(self) -> bool:
        return self.training

    def save(self, path: str, fmt: str = "ghostflw") -> None:
        """Writes the state dict in the GHOSTFLW (default) or safetensors format."""
        from ..io import save_state_dict

        save_state_dict({k: v for k, v in self.state_dict().items()}, path, fmt=fmt)

    def load(self, path: str, strict: bool = True):
        from ..io import load_state_dict

        sd = load_state_dict(path)
        ref = self.state_dict()
        sd = {k: v.to(ref[k].dtype).reshape(ref[k].shape) if k in ref else v for k, v in sd.items()}
        return self.load_state_dict(sd, strict=strict)


class Sequential(Module):
    """Ordered container. ``Sequential([a, b])``, ``Sequential(a, b)`` or ``Sequential().add_layer(a)``."""

    def __init__(self, *layers):
        super().__init__()
        if len(layers) == 1 and isinstance(layers[0], (list, tuple)):
            layers = tuple(layers[0])
        self.layers = torch.nn.ModuleList(layers)

    def add_layer(self, layer):
        self.layers.append(layer)
        return self

    add = add_layer

    def forward(self, x):
        for layer in self.layers:
            x = layer(x)
        return x

    def __len__(self):
        return len(self.layers)

    def __getitem__(self, i):
        return self.layers[i]

    def __iter__(self):
        return iter(self.layers)
