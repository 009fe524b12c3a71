"""Collective back-ends for the training engines.

``make_comm("nccl", device)`` is the baseline: torch.distributed collectives (NCCL on GPUs, gloo on
CPU ranks). ``make_comm("fused", device)`` uses this package's own peer-memory kernels where the
symmetric-memory substrate is available and falls back to the baseline otherwise (it says so once).
"""
from __future__ import annotations

import warnings

import torch.distributed as dist

from .zero3 import Comm


def make_comm(kind: str, device, group=None) -> Comm:
    if not (dist.is_available() and dist.is_initialized()):
        return Comm(None)
    if kind == "fused":
        try:
            from .symm import FusedComm

            return FusedComm(device, group)
        except Exception as e:  # substrate unavailable: say so, use the baseline
            if dist.get_rank() == 0:
                warnings.warn(f"fused peer-memory collectives unavailable ({e!r}); using NCCL")
            return Comm(group)
    return Comm(group)
