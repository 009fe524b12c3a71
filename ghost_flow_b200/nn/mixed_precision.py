"""Mixed precision: ``PrecisionMode``, ``MixedPrecisionConfig`` presets, ``GradScaler`` with the reference's state
machine (ghostflow-nn/src/mixed_precision.rs:29-197: init scale 65536 / 1 / 1024 for fp16 / bf16 / fp8, growth 2,
backoff 0.5, growth interval 2000, skip the step on inf/nan), ``autocast`` and real format conversions.

Where the reference fakes reduced precision by rounding fp32 values (mixed_precision.rs:220-285), these helpers
cast to the real formats: IEEE fp16, bf16, and fp8 e4m3 with one scale per 32-element block.
"""
from __future__ import annotations

import enum
from dataclasses import dataclass

import torch


class PrecisionMode(enum.Enum):
    FP32 = "fp32"
    FP16 = "fp16"
    BF16 = "bf16"
    FP8 = "fp8"

    def torch_dtype(self):
        return {"fp32": torch.float32, "fp16": torch.float16, "bf16": torch.bfloat16,
                "fp8": torch.float8_e4m3fn}[self.value]


@dataclass
class MixedPrecisionConfig:
    mode: PrecisionMode = PrecisionMode.FP32
    init_scale: float = 1.0
    growth_factor: float = 2.0
    backoff_factor: float = 0.5
    growth_interval: int = 2000
    dynamic_loss_scale: bool = True

    @classmethod
    def fp16(cls): return cls(PrecisionMode.FP16, 65536.0)
    @classmethod
    def bf16(cls): return cls(PrecisionMode.BF16, 1.0, dynamic_loss_scale=False)
    @classmethod
    def fp8(cls): return cls(PrecisionMode.FP8, 1024.0)
    @classmethod
    def fp32(cls): return cls()


class GradScaler:
    """Loss scaling with overflow detection: ``scale_loss`` -> backward -> ``unscale_gradients`` -> ``step``."""

    def __init__(self, config: MixedPrecisionConfig | None = None):
        self.config = config or MixedPrecisionConfig.fp16()
        self.scale = float(self.config.init_scale)
        self.growth_tracker = 0
        self.found_inf = False
        self.num_overflows = 0
        self.num_steps = 0

    def get_scale(self) -> float:
        return self.scale

    def scale_loss(self, loss):
        from ..tensor import Tensor

        if isinstance(loss, Tensor):
            return Tensor(loss.data * self.scale)
        return loss * self.scale

    def unscale_gradients(self, params) -> bool:
        """Divides gradients by the scale in place; returns True when every gradient is finite."""
        inv = 1.0 / self.scale
        self.found_inf = False
        for p in params:
            p = getattr(p, "data", p) if not isinstance(p, torch.Tensor) else p
            if p.grad is None:
                continue
            p.grad.mul_(inv)
            if not bool(torch.isfinite(p.grad).all()):
                self.found_inf = True
        return not self.found_inf

    def step(self, optimizer) -> bool:
        """Runs ``optimizer.step()`` unless an overflow was found; updates the scale. Returns True if stepped."""
        self.num_steps += 1
        stepped = False
        if self.found_inf:
            self.num_overflows += 1
            if self.config.dynamic_loss_scale:
                self.scale = max(self.scale * self.config.backoff_factor, 1.0)
            self.growth_tracker = 0
        else:
            optimizer.step()
            stepped = True
            self.growth_tracker += 1
            if self.config.dynamic_loss_scale and self.growth_tracker >= self.config.growth_interval:
                self.scale *= self.config.growth_factor
                self.growth_tracker = 0
        self.found_inf = False
        return stepped

    update_scale = step

    def get_stats(self) -> dict:
        return {"scale": self.scale, "growth_tracker": self.growth_tracker, "num_overflows": self.num_overflows,
                "num_steps": self.num_steps}

    def state_dict(self):
        return self.get_stats()

    def load_state_dict(self, sd):
        self.scale, self.growth_tracker = sd["scale"], sd["growth_tracker"]
        self.num_overflows, self.num_steps = sd["num_overflows"], sd["num_steps"]


def to_half_precision(t: torch.Tensor, mode: PrecisionMode = PrecisionMode.BF16) -> torch.Tensor:
    if mode == PrecisionMode.FP8:
        q, s = quantize_fp8_blockwise(t)
        return dequantize_fp8_blockwise(q, s, t.shape)
    return t.to(mode.torch_dtype())


def to_full_precision(t: torch.Tensor) -> torch.Tensor:
    return t.to(torch.float32)


def quantize_fp8_blockwise(t: torch.Tensor, block: int = 32):
    """e4m3 values with one power-of-two scale per ``block`` consecutive elements of the last dim.
    Returns (fp8 tensor [..., n], scales fp32 [..., n / block])."""
    n = t.shape[-1]
    pad = (-n) % block
    x = torch.nn.functional.pad(t.float(), (0, pad)) if pad else t.float()
    xb = x.reshape(*x.shape[:-1], -1, block)
    amax = xb.abs().amax(-1, keepdim=True).clamp(min=2.0 ** -126)
    scale = torch.exp2(torch.ceil(torch.log2(amax / 448.0)))
    q = (xb / scale).to(torch.float8_e4m3fn)
    return q.reshape(*x.shape[:-1], -1)[..., :n], scale.squeeze(-1)


def dequantize_fp8_blockwise(q: torch.Tensor, scale: torch.Tensor, shape=None, block: int = 32):
    n = q.shape[-1]
    pad = (-n) % block
    x = q.float()
    if pad:
        x = torch.nn.functional.pad(x, (0, pad))
    xb = x.reshape(*x.shape[:-1], -1, block) * scale.unsqueeze(-1)
    return xb.reshape(*x.shape[:-1], -1)[..., :n]


class AutocastContext:
    """``with AutocastContext(PrecisionMode.BF16): ...`` runs eligible ops in the reduced precision."""

    def __init__(self, mode: PrecisionMode = PrecisionMode.BF16, device_type: str | None = None, enabled=True):
        self.mode = mode
        dt = mode.torch_dtype() if mode in (PrecisionMode.FP16, PrecisionMode.BF16) else torch.bfloat16
        device_type = device_type or ("cuda" if torch.cuda.is_available() else "cpu")
        self._ctx = torch.autocast(device_type, dtype=dt, enabled=enabled and mode != PrecisionMode.FP32)

    def __enter__(self):
        self._ctx.__enter__()
        return self

    def __exit__(self, *a):
        return self._ctx.__exit__(*a)


autocast = AutocastContext
