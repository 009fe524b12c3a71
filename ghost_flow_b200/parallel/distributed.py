"""Data / model / pipeline parallel wrappers and the generic ZeRO optimizer, with the reference's names but real
collectives (``torch.distributed``: NCCL on GPUs, gloo on CPU).

Reference: ghostflow-nn/src/distributed.rs (DistributedBackend :11-18, DistributedConfig :35-45, DataParallel :51-139,
ModelParallel :145-184, GradientAccumulator :190-267, DistributedDataParallel :273-329, PipelineParallel :334-391)
and ghostflow-nn/src/zero_optimizer.rs (ZeRoStage/ZeRoConfig :15-55, partitioning :149-195, reduce-scatter :220-242,
all-gather :245-259, step :262-309, offload :312-341, stats :344-404). Every collective there is simulated
(gradients are multiplied by 1/world, parameters cloned); here they move data.

The flagship LLaMA trainer does not go through these wrappers: it has its own hand-scheduled engine
(:mod:`ghost_flow_b200.parallel.zero3`). These classes serve arbitrary ``torch.nn.Module`` models.
"""
from __future__ import annotations

import contextlib
import enum
import math
import os
from dataclasses import dataclass, field

import torch
import torch.distributed as dist

from ..ops import raw


class DistributedBackend(enum.Enum):
    NCCL = "nccl"
    Gloo = "gloo"
    MPI = "mpi"


@dataclass
class DistributedConfig:
    backend: DistributedBackend = DistributedBackend.NCCL
    world_size: int = 1
    rank: int = 0
    master_addr: str = "127.0.0.1"
    master_port: int = 29500

    @classmethod
    def from_env(cls, backend=None):
        be = backend or (DistributedBackend.NCCL if torch.cuda.is_available() else DistributedBackend.Gloo)
        return cls(be, int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("RANK", 0)),
                   os.environ.get("MASTER_ADDR", "127.0.0.1"), int(os.environ.get("MASTER_PORT", 29500)))


def init_process_group(config: DistributedConfig, timeout_s: float | None = None):
    """One process per GPU. Idempotent; returns the default group (or None for world_size 1)."""
    if config.world_size <= 1:
        return None
    if not dist.is_initialized():
        import datetime

        os.environ.setdefault("MASTER_ADDR", config.master_addr)
        os.environ.setdefault("MASTER_PORT", str(config.master_port))
        kw = {}
        if timeout_s is not None:
            kw["timeout"] = datetime.timedelta(seconds=timeout_s)
        if config.backend is DistributedBackend.NCCL and torch.cuda.is_available():
            local = int(os.environ.get("LOCAL_RANK", config.rank % max(1, torch.cuda.device_count())))
            torch.cuda.set_device(local)
            kw["device_id"] = torch.device("cuda", local)
        dist.init_process_group(config.backend.value, rank=config.rank, world_size=config.world_size, **kw)
    return dist.group.WORLD


def _world(group=None):
    if dist.is_available() and dist.is_initialized():
        return dist.get_world_size(group), dist.get_rank(group)
    return 1, 0


# --------------------------------------------------------------------------------------------- data parallel
class DataParallel:
    """Replicated model, batch split along dim 0, gradients averaged over ranks (one all-reduce per tensor, the
    reference's granularity; :class:`DistributedDataParallel` buckets)."""

    def __init__(self, module: torch.nn.Module, device_ids=None, group=None):
        self.module = module
        self.device_ids = list(device_ids) if device_ids is not None else [0]
        self.group = group

    def split_batch(self, batch: torch.Tensor, parts: int | None = None):
        """``parts`` near-equal slices along dim 0 (the last takes the remainder)."""
        parts = parts or len(self.device_ids)
        n = batch.shape[0]
        per = n // parts
        out = []
        for i in range(parts):
            lo = i * per
            hi = n if i == parts - 1 else lo + per
            out.append(batch[lo:hi])
        return out

    def all_reduce_gradients(self, grads: dict | None = None) -> dict:
        """Mean over ranks. ``grads``: name -> tensor; default: the module's ``.grad`` fields (in place)."""
        world, _ = _world(self.group)
        if grads is None:
            grads = {n: p.grad for n, p in self.module.named_parameters() if p.grad is not None}
        for g in grads.values():
            if world > 1:
                dist.all_reduce(g, group=self.group)
                g.div_(world)
        return grads

    def broadcast_parameters(self, src: int = 0):
        world, _ = _world(self.group)
        if world > 1:
            for t in list(self.module.parameters()) + list(self.module.buffers()):
                dist.broadcast(t.data, src, group=self.group)

    def forward(self, *a, **k):
        return self.module(*a, **k)

    __call__ = forward


class GradientAccumulator:
    """Sums gradients over ``accumulation_steps`` micro-steps, hands back the mean."""

    def __init__(self, accumulation_steps: int):
        self.accumulation_steps = accumulation_steps
        self.current_step = 0
        self.accumulated: dict[str, torch.Tensor] = {}

    def accumulate(self, grads: dict) -> bool:
        for n, g in grads.items():
            if n in self.accumulated:
                self.accumulated[n].add_(g)
            else:
                self.accumulated[n] = g.detach().clone()
        self.current_step += 1
        return self.should_step()

    def should_step(self) -> bool:
        return self.current_step >= self.accumulation_steps

    def get_and_reset(self) -> dict:
        out = {n: g / self.accumulation_steps for n, g in self.accumulated.items()}
        self.accumulated, self.current_step = {}, 0
        return out


class DistributedDataParallel(torch.nn.Module):
    """Flat gradient buckets all-reduced asynchronously while backward still runs.

    Parameters are laid into buckets of ``bucket_mb`` in reverse registration order (roughly the order their
    gradients become ready); each parameter's ``.grad`` is a view into its bucket, so no copy precedes the
    collective. A bucket's all-reduce is launched from the hook of its last-arriving gradient. ``finish()`` (called
    by ``step`` helpers or by the user before the optimizer) waits for all of them and divides by the world size."""

    def __init__(self, module: torch.nn.Module, group=None, bucket_mb: float = 25.0, accumulation_steps: int = 1):
        super().__init__()
        self.module = module
        self.group = group
        self.world, self.rank = _world(group)
        self.accumulation_steps = accumulation_steps
        self._micro = 0
        self._sync = True
        self._works = []
        params = [p for p in module.parameters() if p.requires_grad]
        self.buckets: list[torch.Tensor] = []
        self._bucket_of: dict[int, int] = {}
        self._pending: list[int] = []
        cap = int(bucket_mb * (1 << 20))
        cur, cur_bytes = [], 0
        groups = []
        for p in reversed(params):
            nbytes = p.numel() * p.element_size()
            if cur and (cur_bytes + nbytes > cap or cur[0].dtype != p.dtype):
                groups.append(cur)
                cur, cur_bytes = [], 0
            cur.append(p)
            cur_bytes += nbytes
        if cur:
            groups.append(cur)
        for bi, ps in enumerate(groups):
            flat = torch.zeros(sum(p.numel() for p in ps), dtype=ps[0].dtype, device=ps[0].device)
            off = 0
            for p in ps:
                p.grad = flat[off:off + p.numel()].view_as(p)
                off += p.numel()
                self._bucket_of[id(p)] = bi
                p.register_post_accumulate_grad_hook(self._hook)
            self.buckets.append(flat)
            self._pending.append(len(ps))
        self._sizes = list(self._pending)
        self._next = 0
        if self.world > 1:
            DataParallel(module, group=group).broadcast_parameters(0)

    def _hook(self, p):
        bi = self._bucket_of[id(p)]
        self._pending[bi] -= 1
        if self._pending[bi] == 0 and self._sync and self.world > 1:
            self._launch_ready()

    def _launch_ready(self, everything: bool = False):
        """Collectives must be issued in the same order on every rank, and the order in which hooks fire is not
        the same everywhere (a parameter may get no gradient on one rank only). Buckets are therefore launched
        strictly by index: a complete bucket waits until all buckets before it have been launched."""
        while self._next < len(self.buckets) and (everything or self._pending[self._next] <= 0):
            self._works.append(dist.all_reduce(self.buckets[self._next], group=self.group, async_op=True))
            self._next += 1

    @contextlib.contextmanager
    def no_sync(self):
        """Skip the all-reduce for the backward passes inside (gradient accumulation)."""
        old, self._sync = self._sync, False
        try:
            yield
        finally:
            self._sync = old

    def _reset_counts(self):
        self._pending = list(self._sizes)
        self._next = 0      # first bucket whose all-reduce has not been launched in this backward

    def forward(self, *a, **k):
        self._reset_counts()
        return self.module(*a, **k)

    def finish(self):
        """Wait for the bucket all-reduces of the last backward and turn sums into means. A bucket whose
        all-reduce no hook launched is reduced here: that happens when one of its parameters (or of a bucket before
        it) got no gradient in this backward (unused in the forward pass, a branch not taken), because the hook of
        such a parameter never fires; its slice of the bucket holds zeros (or the accumulated value) and takes part
        like any other.
        Without this the ranks would keep their local gradients, scaled by 1 / world, and drift apart."""
        if self.world > 1 and self._sync:
            self._launch_ready(everything=True)
        for w in self._works:
            w.wait()
        self._works = []
        if self.world > 1 and self._sync:
            for b in self.buckets:
                b.div_(self.world)
        # a second backward without a forward in between (two losses) starts from fresh counts as well
        self._reset_counts()

    def zero_grad(self):
        for b in self.buckets:
            b.zero_()

    def backward(self, loss: torch.Tensor) -> bool:
        """The reference's entry point: backward, all-reduce, accumulate; True when an optimizer step is due."""
        self._micro += 1
        last = self._micro % self.accumulation_steps == 0
        self._reset_counts()
        if last:
            (loss / self.accumulation_steps).backward()
            self.finish()
        else:
            with self.no_sync():
                (loss / self.accumulation_steps).backward()
        return last


# --------------------------------------------------------------------------------------------- ZeRO
class ZeRoStage(enum.IntEnum):
    Stage1 = 1      # optimizer state sharded
    Stage2 = 2      # + gradients sharded
    Stage3 = 3      # + parameters sharded


@dataclass
class ZeRoConfig:
    stage: ZeRoStage = ZeRoStage.Stage2
    world_size: int = 1
    rank: int = 0
    cpu_offload: bool = False
    nvme_offload: bool = False
    overlap_comm: bool = True
    bucket_size: int = 25_000_000          # parameters per bucket
    lr: float = 1e-3
    betas: tuple = (0.9, 0.999)
    eps: float = 1e-8
    weight_decay: float = 0.0

    @classmethod
    def default(cls):
        return cls()

    # presets of the reference (ghostflow-nn/src/zero_optimizer.rs:57-110)
    @classmethod
    def stage1(cls, world_size: int = 1, rank: int = 0):
        return cls(stage=ZeRoStage.Stage1, world_size=world_size, rank=rank)

    @classmethod
    def stage2(cls, world_size: int = 1, rank: int = 0):
        return cls(stage=ZeRoStage.Stage2, world_size=world_size, rank=rank)

    @classmethod
    def stage3(cls, world_size: int = 1, rank: int = 0):
        return cls(stage=ZeRoStage.Stage3, world_size=world_size, rank=rank)

    def with_offload(self, cpu: bool = True, nvme: bool = False):
        self.cpu_offload, self.nvme_offload = cpu, nvme
        return self


@dataclass
class ZeRoStats:
    stage: ZeRoStage
    world_size: int
    total_params: int
    owned_params: int
    param_bytes_per_rank: int
    grad_bytes_per_rank: int
    optimizer_bytes_per_rank: int
    offloaded_bytes: int = 0
    # what this implementation keeps allocated on the rank (see ZeRoOptimizer: the flat parameter and gradient
    # buckets stay whole at every stage; only the optimizer state is sharded)
    resident_param_bytes: int = 0
    resident_grad_bytes: int = 0

    def resident_bytes(self) -> int:
        return self.resident_param_bytes + self.resident_grad_bytes + self.optimizer_bytes_per_rank

    def memory_savings_ratio(self) -> float:
        """Bytes of the unsharded mixed-precision state (2 + 2 + 12 per parameter) over this rank's share as the
        STAGE defines it (the reference's formula, ghostflow-nn/src/zero_optimizer.rs:344-368). What this
        implementation really holds is :meth:`resident_bytes`."""
        base = self.total_params * 16
        mine = self.param_bytes_per_rank + self.grad_bytes_per_rank + self.optimizer_bytes_per_rank
        return base / max(1, mine)


@dataclass
class ParameterPartition:
    """Where one parameter lives in the flat partitioning (ghostflow-nn/src/zero_optimizer.rs:96-108). Buckets are
    cut by element ranges, so a tensor can straddle two owners: ``owner_rank`` owns its first element, ``owners``
    lists every rank that owns a part of it."""
    name: str
    owner_rank: int
    start_idx: int          # first element in the flat bucket
    end_idx: int            # one past the last element
    shape: tuple
    bucket: int = 0
    owners: tuple = ()


class ZeRoOptimizer:
    """AdamW with ZeRO partitioning over flat element ranges (not whole tensors as in the reference, whose owner
    map depends on hash-map order).

    All trainable parameters are laid into flat buckets of at most ``bucket_size`` elements, padded to a multiple
    of the world size; rank r owns the r-th slice of every bucket: its fp32 master copy and both moments live
    only there. ``step()``: reduce-scatter of each gradient bucket (mean), fused AdamW on the owned slice (one
    kernel: fp32 update + low-precision copy), all-gather of the updated slices.

    The stages differ in what they are ALLOWED to drop, not in what this class drops: the flat parameter and
    gradient buckets stay allocated whole at every stage (parameters and ``.grad`` are views of them, which is what
    lets the collectives and the fused kernels run on single flat tensors), so the memory this class saves is the
    optimizer state (12 of 16 bytes per parameter), i.e. stage 1. ``get_stats()`` reports both the stage's nominal
    share (the reference's formula) and the bytes really resident. The engine that shards parameters and gradients
    for real is :class:`~ghost_flow_b200.parallel.zero3.Zero3LlamaEngine`.
    """

    # signal-pad layout of the fused path (int32 indices, 8 per bucket, one slot per writer rank)
    _PAD_READY, _PAD_CONSUMED, _PAD_VERSION, _MAX_FUSED_BUCKETS = 1024, 2048, 3072, 128

    def __init__(self, params, config: ZeRoConfig | None = None, group=None, comm: str = "nccl",
                 overlap: bool | None = None, capturable: bool = False):
        """``overlap`` (default: on for CUDA parameters and more than one rank): a bucket's reduce-scatter, AdamW and
        all-gather are launched on a side stream from a gradient hook as soon as the backward pass has produced the
        bucket's last gradient, so they run under the rest of the backward pass; ``step()`` then only launches
        what is left and joins the side stream. With gradient accumulation over several backward passes wrap all
        but the last in ``no_sync()``.

        ``capturable``: the step number lives in a device counter that ``step()`` bumps with a one-thread kernel,
        Adam's bias corrections and the flag values of the fused path are computed from it on the device, and
        nothing in ``zero_grad()`` / backward hooks / ``step()`` reads device memory on the host: forward, backward
        and ``step()`` can be recorded once in a CUDA graph and replayed (``ghost_flow_b200.utils.GraphedStep``).

        ``comm="fused"`` (bf16 CUDA parameters, 2 to 8 ranks of one NVSwitch box): the gradient buckets live
        in symmetric memory and ``step()`` runs, per bucket, ONE kernel that reads this rank's slice of every
        rank's gradients over NVLink, averages it and applies AdamW to the owned shard (``gf_rs_adamw_fused``),
        then a pull all-gather of the updated bf16 shards (``gf_allgather_pull``); ranks order themselves with
        release/acquire flags, every wait is bounded. ``comm="nccl"`` uses reduce-scatter / all-gather collectives
        around the flat AdamW kernel."""
        self.config = config or ZeRoConfig.default()
        self.group = group
        self.world, self.rank = _world(group)
        if self.world == 1:
            self.world, self.rank = 1, 0
        self.params = [p for p in params if p.requires_grad]
        self.step_count = 0
        self.buckets = []
        cuda = bool(self.params) and self.params[0].is_cuda
        # on CPU ranks (gloo) an explicit overlap=True launches the bucket work straight from the hooks (no side
        # stream): nothing overlaps there, but the hook bookkeeping is the same and can be tested without a GPU
        self.overlap = (cuda and self.world > 1) if overlap is None else bool(overlap)
        self.capturable = bool(capturable) and cuda
        self._sync_hooks = True
        self._flag_epoch = 0
        self._open = False
        self._launched: set = set()
        self._side = torch.cuda.Stream(self.params[0].device) if (self.overlap and cuda) else None
        self._step_dev = (torch.zeros(1, dtype=torch.int32, device=self.params[0].device) if self.capturable
                          else None)
        groups, cur, n = [], [], 0
        for p in self.params:
            if cur and (n + p.numel() > self.config.bucket_size or cur[0].dtype != p.dtype):
                groups.append(cur)
                cur, n = [], 0
            cur.append(p)
            n += p.numel()
        if cur:
            groups.append(cur)
        self._fc = None
        if comm == "fused":
            ok = (2 <= self.world <= 8 and len(groups) <= self._MAX_FUSED_BUCKETS
                  and all(p.is_cuda and p.dtype == torch.bfloat16 for p in self.params))
            if not ok:
                raise RuntimeError("comm='fused' needs bf16 CUDA parameters, 2..8 ranks and at most "
                                   f"{self._MAX_FUSED_BUCKETS} buckets")
            from .symm import FusedComm

            self._fc = FusedComm(self.params[0].device, group)
            total = 0
            for g in groups:
                padded = self._padded(sum(p.numel() for p in g))
                total += (padded * 2 + 255) // 256 * 256 + (padded // self.world * 2 + 255) // 256 * 256
            self._fc.reserve(total)
        elif comm != "nccl":
            raise ValueError(f"unknown comm {comm!r}")
        for g in groups:
            self._make_bucket(g)
        self._offloaded = False
        self._pending = [len(b["params"]) for b in self.buckets]
        if self.overlap:
            for i, b in enumerate(self.buckets):
                for prm in b["params"]:
                    prm.register_post_accumulate_grad_hook(self._grad_hook(i))

    # ---- overlap: gradient hooks
    def _grad_hook(self, bucket_index: int):
        def hook(_param):
            if not self._sync_hooks or self._offloaded:
                return
            if bucket_index in self._launched:
                # the bucket was reduced and its shard updated during an earlier backward pass of this step
                raise RuntimeError("a second backward pass reached a bucket that was already reduced and updated in "
                                   "this step: wrap every backward pass but the last in ZeRoOptimizer.no_sync()")
            self._pending[bucket_index] -= 1
            if self._pending[bucket_index] == 0:
                self._launch_bucket(bucket_index)
        return hook

    def no_sync(self):
        """Context manager: backward passes inside it only accumulate gradients (no per-bucket launches)."""
        opt = self

        class _NoSync:
            def __enter__(self):
                opt._sync_hooks = False

            def __exit__(self, *exc):
                opt._sync_hooks = True
        return _NoSync()

    def _begin_step(self):
        if self._open:
            return
        self._open = True
        self.step_count += 1
        self._flag_epoch += 1          # flag values of the fused path: launches of this object, never set back
        if self.capturable:
            from ..ops import _lib

            _lib.check_rc(_lib.cuda_lib().gf_counter_add(self._step_dev.data_ptr(), 1, _lib.stream_ptr()),
                          "gf_counter_add")

    def _launch_bucket(self, i: int):
        """Everything bucket ``i`` needs after its gradients are complete, on the side stream when overlapping."""
        self._begin_step()
        if self._side is not None:
            self._side.wait_event(torch.cuda.current_stream().record_event())
            with torch.cuda.stream(self._side):
                self._bucket_work(i)
        else:
            self._bucket_work(i)
        self._launched.add(i)

    def _bucket_work(self, i: int):
        if self._fc is not None:
            self._bucket_fused(i)
            return
        c, b = self.config, self.buckets[i]
        lo = self.rank * b["shard"]
        # reduce-scatter of the flat gradient
        if self.world == 1:
            g_shard = b["flat_g"][:b["shard"]]
        elif dist.get_backend(self.group) == "nccl":
            dist.reduce_scatter_tensor(b["g_shard"], b["flat_g"], group=self.group)
            g_shard = b["g_shard"]
        else:
            tmp = b["flat_g"].float()
            dist.all_reduce(tmp, group=self.group)
            b["g_shard"].copy_(tmp[lo:lo + b["shard"]].to(b["g_shard"].dtype))
            g_shard = b["g_shard"]
        p_lp = b["flat_p"][lo:lo + b["shard"]]
        kw = dict(lr=c.lr, beta1=c.betas[0], beta2=c.betas[1], eps=c.eps, weight_decay=c.weight_decay,
                  step=self.step_count, grad_scale=1.0 / self.world)
        lp_out = p_lp if p_lp.dtype != torch.float32 else None
        if self.capturable:
            from ..ops.optim_kernels import adam_flat

            adam_flat(b["master"], b["m"], b["v"], g_shard, lp_out, step_dev=self._step_dev, **kw)
        else:
            raw.adamw_flat(b["master"], b["m"], b["v"], g_shard, lp_out, **kw)
        if lp_out is None:
            p_lp.copy_(b["master"])
        if self.world > 1:
            if dist.get_backend(self.group) == "nccl":
                dist.all_gather_into_tensor(b["flat_p"], p_lp, group=self.group)   # in place: p_lp is slice `rank`
            else:
                dist.all_gather_into_tensor(b["flat_p"], p_lp.clone(), group=self.group)

    def _padded(self, n: int) -> int:
        return (n + self.world * 8 - 1) // (self.world * 8) * (self.world * 8)

    def _make_bucket(self, ps):
        dev, dt = ps[0].device, ps[0].dtype
        n = sum(p.numel() for p in ps)
        padded = self._padded(n)
        shard = padded // self.world
        flat_p = torch.zeros(padded, dtype=dt, device=dev)
        if self._fc is not None:
            flat_g = self._fc.alloc(padded, dt)
            shard_lp = self._fc.alloc(shard, dt)
        else:
            flat_g = torch.zeros(padded, dtype=dt, device=dev)
            shard_lp = None
        off = 0
        for p in ps:
            flat_p[off:off + p.numel()].copy_(p.data.reshape(-1))
            p.data = flat_p[off:off + p.numel()].view_as(p)
            p.grad = flat_g[off:off + p.numel()].view_as(p)
            off += p.numel()
        lo = self.rank * shard
        b = {"params": ps, "n": n, "padded": padded, "shard": shard, "flat_p": flat_p, "flat_g": flat_g,
             "master": flat_p[lo:lo + shard].float().clone(), "m": torch.zeros(shard, device=dev),
             "v": torch.zeros(shard, device=dev), "g_shard": torch.zeros(shard, dtype=dt, device=dev),
             "shard_lp": shard_lp}
        if shard_lp is not None:
            shard_lp.copy_(flat_p[lo:lo + shard])
        self.buckets.append(b)

    # ---- partition queries (reference names)
    def partition_parameters(self):
        """[(bucket, first element, last element)] owned by this rank."""
        return [(i, self.rank * b["shard"], (self.rank + 1) * b["shard"]) for i, b in enumerate(self.buckets)]

    def parameter_partitions(self, names=None) -> list:
        """One :class:`ParameterPartition` per parameter, in bucket order. ``names``: optional list of names in the
        order the parameters were given (defaults to ``param<i>``)."""
        out, k = [], 0
        for bi, b in enumerate(self.buckets):
            off = 0
            for p in b["params"]:
                lo, hi = off, off + p.numel()
                first, last = lo // b["shard"], (hi - 1) // b["shard"]
                out.append(ParameterPartition(names[k] if names else f"param{k}", first, lo, hi, tuple(p.shape), bi,
                                              tuple(range(first, last + 1))))
                off = hi
                k += 1
        return out

    def owns(self, bucket: int, element: int) -> bool:
        b = self.buckets[bucket]
        return self.rank * b["shard"] <= element < (self.rank + 1) * b["shard"]

    # ---- collectives
    def reduce_scatter_gradients(self):
        for b in self.buckets:
            if self.world == 1:
                b["g_shard"].copy_(b["flat_g"][:b["shard"]])
                continue
            if dist.get_backend(self.group) == "nccl":
                dist.reduce_scatter_tensor(b["g_shard"], b["flat_g"], group=self.group)
            else:
                tmp = b["flat_g"].float()
                dist.all_reduce(tmp, group=self.group)
                b["g_shard"].copy_(tmp[self.rank * b["shard"]:(self.rank + 1) * b["shard"]].to(b["g_shard"].dtype))

    def all_gather_parameters(self):
        for b in self.buckets:
            if self.world == 1:
                continue
            lo = self.rank * b["shard"]
            dist.all_gather_into_tensor(b["flat_p"], b["flat_p"][lo:lo + b["shard"]].clone(), group=self.group)

    gather_parameters = all_gather_parameters

    def release_parameters(self):
        """Stage 3: after backward only the owned slice has to stay valid (the flat buffer is kept allocated so
        that parameter views stay usable; a rank must not read foreign slices until the next gather)."""

    # ---- step
    def _bucket_fused(self, i: int):
        """Tell the peers that my gradients of bucket ``i`` are complete; one kernel = wait for everybody's
        gradients, sum my slice over peer memory, AdamW on my shard; pull every rank's new bf16 shard into the
        parameter buffer."""
        from ..ops import _lib

        c, fc, b = self.config, self._fc, self.buckets[i]
        W, R = self.world, self.rank
        # flag values: the step number; in capturable mode the launch carries 0 and the device counter adds it
        ep = self._step_dev.data_ptr() if self.capturable else None
        t = 0 if self.capturable else self._flag_epoch
        status, stream = _lib.status_word(fc.device).data_ptr(), _lib.stream_ptr()
        # waits give up after about 2 s; the first step gets about 13 s, since ranks reach it with start-up skew
        limit = (1 << 27) if self._flag_epoch == 1 else 0
        with torch.cuda.device(fc.device):
            _lib.check_rc(fc.lib.gf_signal_peers_ep(fc.pad_ptrs, W, R, self._PAD_READY + 8 * i, t, ep, stream),
                          "gf_signal_peers")
            rc = fc.lib.gf_rs_adamw_fused_ep(
                fc.peer_ptrs(b["flat_g"]), fc.mc_ptr(b["flat_g"]), fc.pad_ptrs, W, R, R * b["shard"], b["shard"],
                b["master"].data_ptr(), b["m"].data_ptr(), b["v"].data_ptr(), b["shard_lp"].data_ptr(),
                float(c.lr), float(c.betas[0]), float(c.betas[1]), float(c.eps), float(c.weight_decay),
                self.step_count, 1.0 / W, self._PAD_READY + 8 * i, t, self._PAD_CONSUMED + 8 * i, t,
                self._PAD_VERSION + 8 * i, t, fc.rs_counter.data_ptr(), 0, limit, status, ep, stream)
            _lib.check_rc(rc, "gf_rs_adamw_fused")
            fc.ag_epoch += 1
            rc = fc.lib.gf_allgather_pull_ep(
                fc.peer_ptrs(b["shard_lp"]), b["flat_p"].data_ptr(), b["shard"], W, R, fc.pad.data_ptr(),
                self._PAD_VERSION + 8 * i, t, fc.ag_ready.data_ptr(), fc.ag_epoch, fc.ag_counters.data_ptr(),
                max(8, 256 // W), limit, status, ep, stream)
            _lib.check_rc(rc, "gf_allgather_pull")

    def _finish_fused(self):
        """Wait until the peers have read my gradients, so that the next backward pass may overwrite them."""
        from ..ops import _lib

        fc = self._fc
        ep = self._step_dev.data_ptr() if self.capturable else None
        t = 0 if self.capturable else self._flag_epoch
        limit = (1 << 27) if self._flag_epoch == 1 else 0
        status, stream = _lib.status_word(fc.device).data_ptr(), _lib.stream_ptr()
        with torch.cuda.device(fc.device):
            for i in range(len(self.buckets)):
                _lib.check_rc(fc.lib.gf_wait_flags_ep(fc.pad.data_ptr(), self._PAD_CONSUMED + 8 * i, self.world, t,
                                                      limit, status, ep, stream), "gf_wait_flags")

    def step(self):
        """Launches what the gradient hooks have not launched yet (every bucket, without overlap), in bucket
        order, and makes the current stream wait for the side stream."""
        if self._offloaded:
            self.load_from_cpu()
        self._begin_step()
        for i in range(len(self.buckets)):
            if i not in self._launched:
                self._launch_bucket(i)
        if self._side is not None:
            if self._fc is not None:
                with torch.cuda.stream(self._side):
                    self._finish_fused()
            torch.cuda.current_stream().wait_event(self._side.record_event())
        elif self._fc is not None:
            self._finish_fused()
        self._launched = set()
        self._pending = [len(b["params"]) for b in self.buckets]
        self._open = False
        if self.config.cpu_offload:
            self.offload_to_cpu()

    def zero_grad(self):
        for b in self.buckets:
            b["flat_g"].zero_()

    # ---- offload (real device <-> pinned host copies of the optimizer state shard)
    def offload_to_cpu(self):
        if self._offloaded:
            return
        for b in self.buckets:
            for k in ("master", "m", "v"):
                t = b[k]
                if t.is_cuda:
                    host = torch.empty(t.shape, dtype=t.dtype, pin_memory=True)
                    host.copy_(t, non_blocking=True)
                    b[k + "_dev"] = t.device
                    b[k] = host
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        self._offloaded = True

    def load_from_cpu(self):
        for b in self.buckets:
            for k in ("master", "m", "v"):
                if k + "_dev" in b:
                    b[k] = b[k].to(b.pop(k + "_dev"), non_blocking=True)
        self._offloaded = False

    def get_stats(self) -> ZeRoStats:
        total = sum(b["n"] for b in self.buckets)
        owned = sum(b["shard"] for b in self.buckets)
        esz = self.buckets[0]["flat_p"].element_size() if self.buckets else 2
        st = self.config.stage
        off = sum(b[k].numel() * 4 for b in self.buckets for k in ("master", "m", "v") if not b[k].is_cuda
                  and self.buckets[0]["flat_p"].is_cuda)
        padded = sum(b["padded"] for b in self.buckets)
        return ZeRoStats(st, self.world, total, owned,
                         (owned if st >= ZeRoStage.Stage3 else total) * esz,
                         (owned if st >= ZeRoStage.Stage2 else total) * esz, owned * 12, off,
                         resident_param_bytes=padded * esz, resident_grad_bytes=padded * esz)

    def memory_savings_ratio(self) -> float:
        return self.get_stats().memory_savings_ratio()

    def state_dict(self):
        return {"step": self.step_count,
                "buckets": [{k: b[k].detach().cpu() for k in ("master", "m", "v")} for b in self.buckets]}

    def load_state_dict(self, sd):
        if self.capturable:
            # the device counter is both Adam's step number and the flag value of the fused path: it may only grow
            if self._fc is not None and int(sd["step"]) < self.step_count:
                raise RuntimeError("a capturable fused optimizer cannot go back to an earlier step; load into a new one")
            self._step_dev.fill_(int(sd["step"]))
        self.step_count = sd["step"]
        for b, s in zip(self.buckets, sd["buckets"]):
            for k in ("master", "m", "v"):
                b[k].copy_(s[k])
            lo = self.rank * b["shard"]
            b["flat_p"][lo:lo + b["shard"]].copy_(b["master"].to(b["flat_p"].dtype))
            if b.get("shard_lp") is not None:
                b["shard_lp"].copy_(b["flat_p"][lo:lo + b["shard"]])
        self.all_gather_parameters()


# --------------------------------------------------------------------------------------------- model parallel
class ModelParallel:
    """Layer placement over devices with real transfers between them."""

    def __init__(self, devices):
        self.devices = [torch.device(d) for d in devices]
        self.layer_placement: dict[str, torch.device] = {}

    def place_layer(self, name: str, device_index: int, module: torch.nn.Module | None = None):
        self.layer_placement[name] = self.devices[device_index]
        if module is not None:
            module.to(self.devices[device_index])

    def auto_place_layers(self, layers):
        """Contiguous runs of near-equal length. ``layers``: names or (name, module) pairs."""
        items = [(l, None) if isinstance(l, str) else l for l in layers]
        per = math.ceil(len(items) / len(self.devices))
        for i, (name, mod) in enumerate(items):
            self.place_layer(name, min(i // per, len(self.devices) - 1), mod)
        return dict(self.layer_placement)

    def get_device(self, name: str):
        return self.layer_placement.get(name)

    def transfer(self, t: torch.Tensor, to_layer: str) -> torch.Tensor:
        return t.to(self.layer_placement[to_layer], non_blocking=True)


# --------------------------------------------------------------------------------------------- pipeline parallel
class PipelineParallel:
    """One pipeline stage per rank, 1F1B schedule, activations and their gradients over point-to-point send/recv
    (NCCL on GPUs by design; gloo on CPU).

    ``stage`` is this rank's module. ``run(micro_inputs, loss_fn, targets)``: the first stage feeds
    ``micro_inputs`` (a list of tensors), the last stage computes ``loss_fn(out, target)``; gradients accumulate
    in the stage's parameters. Returns the mean loss on the last stage (None elsewhere).
    ``activation_shape(micro_batch_rows)`` must give the shape of the tensor crossing every stage boundary."""

    def __init__(self, stage: torch.nn.Module, num_micro_batches: int, activation_shape, dtype=torch.float32,
                 device=None, group=None):
        self.stage = stage
        self.num_micro_batches = num_micro_batches
        self.group = group
        self.num_stages, self.stage_index = _world(group)
        self.activation_shape = activation_shape
        self.dtype = dtype
        self.device = device or next(stage.parameters()).device
        self.current_stage = 0

    # reference bookkeeping API
    def create_micro_batches(self, batch: torch.Tensor):
        return list(batch.chunk(self.num_micro_batches, 0))

    def next_stage(self):
        self.current_stage = (self.current_stage + 1) % max(1, self.num_stages)
        return self.current_stage

    @property
    def is_first(self):
        return self.stage_index == 0

    @property
    def is_last(self):
        return self.stage_index == self.num_stages - 1

    # -- point-to-point plumbing ------------------------------------------------------------------------------
    # Every exchange with a neighbour goes out as ONE batch of sends and receives. On NCCL the operations of a batch
    # run as one grouped kernel, so "send the activation forward, receive a gradient back" cannot deadlock against the
    # neighbour's mirrored pair the way two ordered blocking kernels on one stream would for messages larger than
    # NCCL's staging buffers. A batch that only sends is not waited for until the end of the step (the tensor is kept
    # alive), so the transfer overlaps the next micro-batch's compute; a batch that receives is waited for right
    # where its tensor is needed.
    def _exchange(self, send_fwd=None, send_bwd=None, recv_fwd=False, recv_bwd=False, rows=0):
        ops, got_f, got_b = [], None, None
        r = self.stage_index
        rank_of = (lambda i: dist.get_global_rank(self.group, i)) if self.group is not None else (lambda i: i)
        if send_fwd is not None:
            ops.append(dist.P2POp(dist.isend, send_fwd, rank_of(r + 1), self.group))
        if send_bwd is not None:
            ops.append(dist.P2POp(dist.isend, send_bwd, rank_of(r - 1), self.group))
        if recv_fwd:
            got_f = torch.empty(self.activation_shape(rows), dtype=self.dtype, device=self.device)
            ops.append(dist.P2POp(dist.irecv, got_f, rank_of(r - 1), self.group))
        if recv_bwd:
            got_b = torch.empty(self.activation_shape(rows), dtype=self.dtype, device=self.device)
            ops.append(dist.P2POp(dist.irecv, got_b, rank_of(r + 1), self.group))
        if not ops:
            return None, None
        works = dist.batch_isend_irecv(ops)
        if recv_fwd or recv_bwd:
            for w in works:
                w.wait()
            self.p2p_batches_waited += 1
        else:
            self._sends.append((works, send_fwd, send_bwd))
        self.p2p_batches += 1
        return got_f, got_b

    def _forward(self, x_in, i, micro_inputs, saved):
        if self.is_first:
            inp, x = None, micro_inputs[i]
        else:
            inp = x_in.requires_grad_(True)
            x = inp
        out = self.stage(x)
        saved.append((inp, out))
        return None if self.is_last else out.detach().contiguous()

    def _backward(self, g_in, saved, loss_fn, targets, losses, j):
        inp, out = saved.pop(0)
        if self.is_last:
            loss = loss_fn(out, targets[j]) / self.num_micro_batches
            losses.append(loss.detach() * self.num_micro_batches)
            loss.backward()
        else:
            out.backward(g_in)
        return None if self.is_first else inp.grad.contiguous()

    def run(self, micro_inputs=None, loss_fn=None, targets=None, rows: int | None = None):
        m, s, r = self.num_micro_batches, self.num_stages, self.stage_index
        if rows is None:
            rows = micro_inputs[0].shape[0]
        saved, losses = [], []
        self._sends = []
        self.p2p_batches = self.p2p_batches_waited = 0
        if s == 1:
            for i in range(m):
                out = self.stage(micro_inputs[i])
                loss = loss_fn(out, targets[i]) / m
                loss.backward()
                losses.append(loss.detach() * m)
            return torch.stack(losses).mean()
        first, last = self.is_first, self.is_last
        warm = min(m, s - 1 - r)
        steady = m - warm
        f = b = 0
        # warm-up forwards: receive, compute, send on
        for _ in range(warm):
            x, _ = self._exchange(recv_fwd=not first, rows=rows)
            act = self._forward(x, f, micro_inputs, saved)
            f += 1
            self._exchange(send_fwd=act)
        x = self._exchange(recv_fwd=not first, rows=rows)[0] if steady else None
        # steady state: forward, (send activation | receive gradient), backward, (send gradient | receive activation)
        for k in range(steady):
            act = self._forward(x, f, micro_inputs, saved)
            f += 1
            _, g = self._exchange(send_fwd=act, recv_bwd=not last, rows=rows)
            dx = self._backward(g, saved, loss_fn, targets, losses, b)
            b += 1
            more = k + 1 < steady
            x, _ = self._exchange(send_bwd=dx, recv_fwd=more and not first, rows=rows)
        # cool-down backwards
        for _ in range(warm):
            _, g = self._exchange(recv_bwd=not last, rows=rows)
            dx = self._backward(g, saved, loss_fn, targets, losses, b)
            b += 1
            self._exchange(send_bwd=dx)
        for works, *_ in self._sends:
            for w in works:
                w.wait()
        self._sends = []
        return torch.stack(losses).mean() if self.is_last else None
