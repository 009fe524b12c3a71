"""Guard words around the carve-outs of the peer-mapped arenas and kernel workspaces.

The kernels of this package index into a few large buffers that are carved into tensors by offset (the symmetric
arena of the ZeRO path, the tensor-parallel and expert-parallel workspaces). A kernel that runs past the end of its
carve-out lands in a neighbour's data and nothing faults. Every carve-out is therefore followed by 256 bytes of a
fixed pattern, the arena starts with such a block too, and :func:`check_all` (called by the test fixture after
every GPU test and by ``ops._lib.check_status``) compares them all and names the first damaged one with the
offset of its first wrong byte. The check is a few small device comparisons and one host read, so it belongs
between steps or after a test, not inside a step.

No counterpart in the reference (its device memory is a Vec<u8> pool, ghostflow-cuda/src/memory.rs).
"""
from __future__ import annotations

import weakref

import torch

CANARY_BYTES = 256
PATTERN = 0xA5
SLACK_BYTES = 64 * 1024          # room for the guard blocks of up to 255 carve-outs; constructors reserve it on top

_LEDGERS: "weakref.WeakSet[CanaryLedger]" = weakref.WeakSet()


class CanaryError(RuntimeError):
    pass


class CanaryLedger:
    """Guard blocks of one uint8 buffer. ``plant(offset, name)`` writes the pattern at ``[offset, offset + 256)``
    and returns the offset after it."""

    def __init__(self, buf: torch.Tensor, owner: str):
        assert buf.dtype == torch.uint8
        self.buf, self.owner = buf, owner
        self.blocks: list = []          # (offset, name of the carve-out in front of it)
        _LEDGERS.add(self)

    def plant(self, offset: int, name: str) -> int:
        if offset + CANARY_BYTES > self.buf.numel():
            raise RuntimeError(f"{self.owner}: no room for the guard block after {name}")
        self.buf[offset:offset + CANARY_BYTES].fill_(PATTERN)
        self.blocks.append((offset, name))
        return offset + CANARY_BYTES

    def check(self) -> None:
        if not self.blocks:
            return
        views = torch.stack([self.buf[o:o + CANARY_BYTES] for o, _ in self.blocks])
        bad = (views != PATTERN)
        if bool(bad.any()):
            i = int(bad.any(1).nonzero()[0])
            j = int(bad[i].nonzero()[0])
            off, name = self.blocks[i]
            raise CanaryError(f"{self.owner}: guard block after '{name}' damaged at arena byte {off + j} "
                              f"({int(bad[i].sum())} of {CANARY_BYTES} bytes overwritten): a kernel wrote past the end "
                              f"of that carve-out (or before the start of the next one)")


def check_all() -> int:
    """Checks every live ledger; returns how many guard blocks were compared."""
    n = 0
    for led in list(_LEDGERS):
        led.check()
        n += len(led.blocks)
    return n
