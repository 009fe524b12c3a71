"""Peer-memory ("symmetric") collectives for the ZeRO engine: this package's own kernels instead of NCCL.

Every rank reserves one arena in symmetric memory (same size and layout on every rank, every peer's copy
mapped into this rank's address space, plus a small signal pad of flags). Weight shards and the two
gradient staging buffers are carved out of the arena, so that

  * the parameter all-gather is a kernel that pulls the peers' shards over NVLink
    (``gf_allgather_pull``), and
  * the gradient reduce-scatter is fused with the AdamW update: one kernel reads this rank's slice of every
    rank's gradient buffer (peer loads, or ``multimem.ld_reduce`` through the switch when
    ``GF_MULTIMEM=1`` and a multicast mapping exists), sums in fp32 and updates the fp32 master / moments /
    bf16 weights of the shard (``gf_rs_adamw_fused``).

Ordering between ranks uses release/acquire flags in the signal pad; every device-side wait is bounded and
reports through the kernel status word. The arena allocation and handle exchange use
``torch.distributed._symmetric_memory`` (CUDA VMM + NVLink peer mappings); the data path is ours.

The reference has no communication backend at all (ghostflow-nn/src/distributed.rs:104-138,
zero_optimizer.rs:220-259 simulate every collective in-process).
"""
from __future__ import annotations

import ctypes
import os

import torch
import torch.distributed as dist

from ..ops import _lib
from .zero3 import Comm

# signal-pad layout (int32 indices); writer rank r writes at [base + r] of the reader's pad
PAD_READY = 0        # + slot * 8 + src : gradient buffer `slot` of rank src is complete (value = use count)
PAD_CONSUMED = 16    # + slot * 8 + src : rank src has finished reading my gradient buffer `slot`
PAD_VERSION = 64     # + unit * 8 + src : rank src's weight shard of `unit` has been through `value` fused updates
                     #                    of THIS process group's lifetime (not the optimizer step: a job resumed
                     #                    from a checkpoint starts with zeroed pads and step_count = N)
PAD_INTS = 4096


def _u64_array(vals):
    return (ctypes.c_ulonglong * len(vals))(*[int(v) for v in vals])


class FusedComm(Comm):
    """Own-kernel collectives over symmetric memory. Falls back to nothing: construction raises when the
    substrate is missing, and the caller decides (see ``parallel.comm.make_comm``)."""

    fused = True

    def __init__(self, device, group=None):
        super().__init__(group)
        if self.world < 2:
            raise RuntimeError("FusedComm needs at least two ranks")
        if self.world > 8:
            raise RuntimeError("FusedComm covers one NVSwitch box (up to 8 ranks)")
        import torch.distributed._symmetric_memory as symm_mem

        self._symm = symm_mem
        self.device = torch.device(device)
        self.group_name = (group or dist.group.WORLD).group_name
        self.arena = None
        self.offset = 0
        self.use_multimem = os.environ.get("GF_MULTIMEM", "0") == "1"
        self.lib = _lib.cuda_lib()
        self._bind()
        # pad + local flags
        self.pad = symm_mem.empty(PAD_INTS, dtype=torch.int32, device=self.device)
        self.pad.zero_()
        self.pad_hdl = symm_mem.rendezvous(self.pad, self.group_name)
        self.pad_ptrs = _u64_array(self.pad_hdl.buffer_ptrs)
        self.ag_ready = torch.zeros(8, dtype=torch.int32, device=self.device)
        self.ag_counters = torch.zeros(8, dtype=torch.int32, device=self.device)
        self.rs_counter = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.slot_use = [0, 0]
        self.ag_epoch = 0
        # Fused updates launched so far per unit. Every rank launches the same sequence, so this local count is
        # also the version that a gather launched now must see in the peers' shards.
        self.unit_updates: dict[int, int] = {}
        # dry_run = True keeps every kernel of the step except the traffic between ranks (local shard copy, local
        # AdamW on the unreduced gradient slice). The numbers it produces are wrong on purpose: it exists only to
        # time the compute-only step, so that exposed communication = full step - dry step can be reported.
        self.dry_run = False
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)

    def _bind(self):
        P, I, L, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float
        lib = self.lib
        lib.gf_signal_peers.argtypes = [P, I, I, I, I, P]
        lib.gf_wait_flags.argtypes = [P, I, I, I, L, P, P]
        lib.gf_rs_adamw_fused.argtypes = [P, ctypes.c_ulonglong, P, I, I, L, L, P, P, P, P, F, F, F, F, F, I, F,
                                          I, I, I, I, I, I, P, I, L, P, P]
        lib.gf_allgather_pull.argtypes = [P, P, L, I, I, P, I, I, P, I, P, I, L, P, P]
        lib.gf_rs_reduce_only.argtypes = [P, ctypes.c_ulonglong, P, I, I, L, L, P, P, F, I, I, I, I, P, I, L, P, P]
        lib.gf_signal_peers_ep.argtypes = [P, I, I, I, I, P, P]
        lib.gf_wait_flags_ep.argtypes = [P, I, I, I, L, P, P, P]
        lib.gf_rs_adamw_fused_ep.argtypes = [P, ctypes.c_ulonglong, P, I, I, L, L, P, P, P, P, F, F, F, F, F, I, F,
                                             I, I, I, I, I, I, P, I, L, P, P, P]
        lib.gf_allgather_pull_ep.argtypes = [P, P, L, I, I, P, I, I, P, I, P, I, L, P, P, P]
        for fn in (lib.gf_signal_peers, lib.gf_wait_flags, lib.gf_rs_adamw_fused, lib.gf_allgather_pull,
                   lib.gf_rs_reduce_only, lib.gf_signal_peers_ep, lib.gf_wait_flags_ep, lib.gf_rs_adamw_fused_ep,
                   lib.gf_allgather_pull_ep):
            fn.restype = I

    # ------------------------------------------------------------------ arena
    def reserve(self, nbytes: int) -> None:
        """Allocates the symmetric arena (collective call: every rank passes the same size)."""
        from .canary import SLACK_BYTES, CanaryLedger

        nbytes = (nbytes + SLACK_BYTES + 4095) // 4096 * 4096
        if os.environ.get("GF_SYMM_ALLOC", "torch") == "own":
            # the library's own allocator (csrc/symm_alloc.cpp: cuMemCreate / export / import / map of every rank's
            # allocation); no in-switch multicast mapping on this path
            from .symm_alloc import SymmetricAllocation

            job = [os.urandom(4).hex() if self.rank == 0 else None]
            dist.broadcast_object_list(job, src=dist.get_global_rank(self.group, 0) if self.group is not None else 0,
                                       group=self.group)
            self._own = SymmetricAllocation(nbytes, self.rank, self.world, device=self.device.index or 0, job=job[0])
            self.arena = self._own.tensor()[:nbytes]
            self.arena.zero_()
            torch.cuda.synchronize(self.device)
            dist.barrier(group=self.group)
            self.arena_hdl = None
            self.arena_ptrs = list(self._own.ptrs)
            mc = 0
        else:
            self.arena = self._symm.empty(nbytes, dtype=torch.uint8, device=self.device)
            self.arena_hdl = self._symm.rendezvous(self.arena, self.group_name)
            self.arena_ptrs = [int(p) for p in self.arena_hdl.buffer_ptrs]
            mc = getattr(self.arena_hdl, "multicast_ptr", 0) or 0
        self.arena_mc = int(mc) if self.use_multimem else 0
        # guard blocks in front of the first carve-out and behind every carve-out (each rank guards its own copy)
        self.canaries = CanaryLedger(self.arena, f"symmetric arena of rank {self.rank}")
        self.offset = self.canaries.plant(0, "start of the arena")

    def alloc(self, numel: int, dtype, device=None) -> torch.Tensor:
        """Carves a zero-filled tensor out of the arena (same offset on every rank)."""
        esz = torch.empty((), dtype=dtype).element_size()
        nbytes = (numel * esz + 255) // 256 * 256
        if self.arena is None or self.offset + nbytes + 256 > self.arena.numel():
            raise RuntimeError("symmetric arena exhausted; reserve() more")
        t = self.arena[self.offset:self.offset + numel * esz].view(dtype)
        t._gf_arena_offset = self.offset
        t.zero_()
        self.offset = self.canaries.plant(self.offset + nbytes, f"carve-out {len(self.canaries.blocks)} "
                                                                f"({numel} x {str(dtype).replace('torch.', '')})")
        return t

    def peer_ptrs(self, t: torch.Tensor):
        off = t.data_ptr() - self.arena.data_ptr()
        return _u64_array([p + off for p in self.arena_ptrs])

    def mc_ptr(self, t: torch.Tensor) -> int:
        if not self.arena_mc:
            return 0
        return self.arena_mc + (t.data_ptr() - self.arena.data_ptr())

    # ------------------------------------------------------------------ collectives
    def all_gather_unit(self, unit, unit_index: int, full: torch.Tensor, need_version: int | None = None) -> None:
        """Pulls every rank's shard of ``unit`` into ``full`` on the current stream. The copy of rank r's shard
        waits until r has published the version this rank expects: the number of fused updates of the unit
        launched so far (``need_version`` overrides it)."""
        if need_version is None:
            need_version = self.unit_updates.get(unit_index, 0)
        if self.dry_run:
            full[self.rank * unit.shard_numel:(self.rank + 1) * unit.shard_numel].copy_(unit.shard)
            return
        self.ag_epoch += 1
        rc = self.lib.gf_allgather_pull(
            self.peer_ptrs(unit.shard), full.data_ptr(), unit.shard_numel, self.world, self.rank,
            self.pad.data_ptr(), PAD_VERSION + unit_index * 8, need_version, self.ag_ready.data_ptr(),
            self.ag_epoch, self.ag_counters.data_ptr(), max(8, 256 // self.world), 0, _lib.status_word(self.device).data_ptr(),
            _lib.stream_ptr())
        _lib.check_rc(rc, "gf_allgather_pull")

    def grads_ready(self, slot: int) -> None:
        """Called on the compute stream after the last gradient write into buffer ``slot``."""
        if self.dry_run:
            return
        self.slot_use[slot] += 1
        rc = self.lib.gf_signal_peers(self.pad_ptrs, self.world, self.rank, PAD_READY + slot * 8,
                                      self.slot_use[slot], _lib.stream_ptr())
        _lib.check_rc(rc, "gf_signal_peers")

    def wait_grad_slot_free(self, slot: int) -> None:
        """Called on the compute stream before the first gradient write of a new use of buffer ``slot``:
        every peer must have finished reading the previous contents."""
        if self.slot_use[slot] == 0 or self.dry_run:
            return
        rc = self.lib.gf_wait_flags(self.pad.data_ptr(), PAD_CONSUMED + slot * 8, self.world, self.slot_use[slot],
                                    0, _lib.status_word(self.device).data_ptr(), _lib.stream_ptr())
        _lib.check_rc(rc, "gf_wait_flags")

    def reduce_scatter_adamw(self, unit, unit_index: int, g_full: torch.Tensor, slot: int, *, lr, beta1, beta2, eps,
                             weight_decay, step, grad_scale=1.0) -> None:
        """Fused reduce-scatter + AdamW for this rank's shard of ``unit`` on the current stream."""
        if self.dry_run:
            from ..ops import raw as K

            K.adamw_flat(unit.master, unit.m, unit.v, g_full[unit.lo:unit.lo + unit.shard_numel], unit.shard, lr=lr,
                         beta1=beta1, beta2=beta2, eps=eps, weight_decay=weight_decay, step=step,
                         grad_scale=grad_scale)
            return
        use = self.slot_use[slot]
        version = self.unit_updates.get(unit_index, 0) + 1
        self.unit_updates[unit_index] = version
        rc = self.lib.gf_rs_adamw_fused(
            self.peer_ptrs(g_full), self.mc_ptr(g_full), self.pad_ptrs, self.world, self.rank, unit.lo,
            unit.shard_numel, unit.master.data_ptr(), unit.m.data_ptr(), unit.v.data_ptr(), unit.shard.data_ptr(),
            float(lr), float(beta1), float(beta2), float(eps), float(weight_decay), int(step), float(grad_scale),
            PAD_READY + slot * 8, use, PAD_CONSUMED + slot * 8, use, PAD_VERSION + unit_index * 8, version,
            self.rs_counter.data_ptr(), 0, 0, _lib.status_word(self.device).data_ptr(), _lib.stream_ptr())
        _lib.check_rc(rc, "gf_rs_adamw_fused")

    def reduce_only(self, unit, unit_index: int, g_full: torch.Tensor, slot: int, grad_out: torch.Tensor,
                    sumsq: torch.Tensor, grad_scale: float = 1.0) -> None:
        """Reduce-scatter without the update: this rank's slice of every rank's gradient buffer, summed in fp32,
        lands in ``grad_out`` (fp32 [shard_numel]) and the sum of its squares is added to ``sumsq`` (a device
        float). Used when the step needs the global gradient norm before it may touch the weights."""
        if self.dry_run:
            grad_out.copy_(g_full[unit.lo:unit.lo + unit.shard_numel].float() * grad_scale)
            sumsq.add_(grad_out.square().sum())
            return
        use = self.slot_use[slot]
        rc = self.lib.gf_rs_reduce_only(
            self.peer_ptrs(g_full), self.mc_ptr(g_full), self.pad_ptrs, self.world, self.rank, unit.lo,
            unit.shard_numel, grad_out.data_ptr(), sumsq.data_ptr(), float(grad_scale), PAD_READY + slot * 8, use,
            PAD_CONSUMED + slot * 8, use, self.rs_counter.data_ptr(), 0, 0,
            _lib.status_word(self.device).data_ptr(), _lib.stream_ptr())
        _lib.check_rc(rc, "gf_rs_reduce_only")

    def publish_version(self, unit_index: int) -> None:
        """After an update of this rank's shard of ``unit_index`` that was NOT done by the fused reducer (the
        deferred AdamW of a clipped step): tells every peer that the shard holds the next version, on the current
        stream, behind the kernels that wrote it."""
        version = self.unit_updates.get(unit_index, 0) + 1
        self.unit_updates[unit_index] = version
        if self.dry_run:
            return
        rc = self.lib.gf_signal_peers(self.pad_ptrs, self.world, self.rank, PAD_VERSION + unit_index * 8, version,
                                      _lib.stream_ptr())
        _lib.check_rc(rc, "gf_signal_peers")
