"""Tensor parallelism with compute and collective fused into one kernel (one NVSwitch box, up to 8 ranks).

Megatron-style sequence-parallel layout: activations between blocks are sharded over tokens
(``[T / world, hidden]`` per rank).

* ``ColumnParallelLinear``: ``y_local[T, out / world] = all_gather(x)[T, in] @ W_local^T``. The all-gather of the
  token shards and the GEMM run as ONE kernel (``gf_gemm_bf16_allgather``): a few CTAs drive the bulk-copy engine
  to pull the peers' shards into local memory while the other CTAs run tcgen05 tiles on the shards that have
  already landed, starting with this rank's own rows.
* ``RowParallelLinear``: ``y[T / world, out] = reduce_scatter(x_local[T, in / world] @ W_local^T)``. The GEMM epilogue
  stores each partial tile into the owner rank's staging buffer over NVLink and the same kernel reduces the
  arrived partials (``gf_gemm_bf16_reduce_scatter``).

Both have an NCCL path (``fused=False``) that is the baseline and the test oracle. The reference has no tensor
parallelism at all (ghostflow-nn/src/distributed.rs has only simulated data, model and pipeline wrappers).
"""
from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from ..ops import _lib
from ..ops.gemm import gemm_raw

_BOUND = False


def _bind():
    global _BOUND
    lib = _lib.cuda_lib()
    if not _BOUND:
        P, I, L, F, U = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float, ctypes.c_ulonglong
        lib.gf_gemm_bf16_allgather.argtypes = [P, P, P, I, I, I, L, L, L, I, P, P, L, F, P, I, P, P, L, I, I, I, I,
                                               P, P, I, P, I, I, P]
        lib.gf_gemm_bf16_allgather.restype = I
        lib.gf_gemm_bf16_reduce_scatter.argtypes = [P, P, P, I, I, I, L, L, L, P, P, L, F, P, P, P, I, I, I, I, P]
        lib.gf_gemm_bf16_reduce_scatter.restype = I
        _BOUND = True
    return lib


def _u64(vals):
    return (ctypes.c_ulonglong * len(vals))(*[int(v) for v in vals])


class SymmetricWorkspace:
    """A symmetric (peer-mapped) allocation plus its peers' addresses, from ``torch.distributed._symmetric_memory``."""

    def __init__(self, nbytes: int, device, group=None):
        import torch.distributed._symmetric_memory as symm_mem

        self.group = group or dist.group.WORLD
        self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        from .canary import SLACK_BYTES, CanaryLedger

        nbytes = (nbytes + SLACK_BYTES + 4095) // 4096 * 4096
        self.buf = symm_mem.empty(nbytes, dtype=torch.uint8, device=device)
        self.buf.zero_()
        self.hdl = symm_mem.rendezvous(self.buf, self.group.group_name)
        self.ptrs = [int(p) for p in self.hdl.buffer_ptrs]
        # guard blocks: one in front of the first carve-out, one behind every carve-out (each rank guards its own copy)
        self.canaries = CanaryLedger(self.buf, f"symmetric workspace of rank {self.rank}")
        self.offset = self.canaries.plant(0, "start of the workspace")
        torch.cuda.synchronize(device)
        dist.barrier(group=self.group)

    def alloc(self, numel: int, dtype) -> torch.Tensor:
        esz = torch.empty((), dtype=dtype).element_size()
        nbytes = (numel * esz + 255) // 256 * 256
        if self.offset + nbytes + 256 > self.buf.numel():
            raise RuntimeError("symmetric workspace exhausted")
        t = self.buf[self.offset:self.offset + numel * esz].view(dtype)
        # the guard block starts at the next 256-byte boundary behind the tensor (same offsets on every rank)
        self.offset = self.canaries.plant(self.offset + nbytes, f"carve-out {len(self.canaries.blocks)} "
                                                                f"({numel} x {str(dtype).replace('torch.', '')})")
        return t

    def peer_ptrs(self, t: torch.Tensor):
        off = t.data_ptr() - self.buf.data_ptr()
        return [p + off for p in self.ptrs]


class AllGatherGemm:
    """``out[T, N] = all_gather(x_shard)[T, K] @ w[N, K]^T`` in one kernel. ``x_shard`` is ``[T / world, K]``.

    No host synchronisation: a rank publishes its shard with a release flag in every peer's signal pad, and the
    copy CTAs of the kernel wait (bounded) for the owner's flag before pulling a shard. Shards and flags are
    double-buffered by call parity, which is enough because a rank can be at most one call ahead of a peer that
    it exchanges data with in every call."""

    def __init__(self, tokens: int, k: int, device, group=None, copy_ctas: int = 16):
        self.group = group or dist.group.WORLD
        self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        assert tokens % self.world == 0
        self.T, self.K, self.copy_ctas = tokens, k, copy_ctas
        self.shard_elems = tokens // self.world * k
        assert self.shard_elems % 8 == 0
        self.ws = SymmetricWorkspace(2 * self.shard_elems * 2 + 8192, device, self.group)
        self.shards = [self.ws.alloc(self.shard_elems, torch.bfloat16).view(tokens // self.world, k) for _ in range(2)]
        self.src = [_u64(self.ws.peer_ptrs(s)) for s in self.shards]
        self.pad = self.ws.alloc(64, torch.int32)
        self.pad_ptrs = _u64(self.ws.peer_ptrs(self.pad))
        self.full = torch.empty(tokens, k, dtype=torch.bfloat16, device=device)
        self.ready = torch.zeros(8, dtype=torch.int32, device=device)
        self.counters = torch.zeros(8, dtype=torch.int32, device=device)
        self.epoch = 0
        self.device = torch.device(device)

    def __call__(self, x_shard: torch.Tensor, w: torch.Tensor, bias=None, out=None):
        lib = _bind()
        self.epoch += 1
        par = self.epoch & 1
        self.shards[par].copy_(x_shard)
        lib.gf_signal_peers.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                        ctypes.c_void_p]
        _lib.check_rc(lib.gf_signal_peers(self.pad_ptrs, self.world, self.rank, par * 8, self.epoch,
                                          _lib.stream_ptr()), "gf_signal_peers")
        N = w.shape[0]
        if out is None:
            out = torch.empty(self.T, N, dtype=torch.bfloat16, device=self.device)
        rc = lib.gf_gemm_bf16_allgather(
            self.full.data_ptr(), w.data_ptr(), out.data_ptr(), self.T, N, self.K, self.full.stride(0), w.stride(0),
            out.stride(0), 0, bias.data_ptr() if bias is not None else None, None, 0, 1.0,
            _lib.status_word(self.device).data_ptr(), 0, self.src[par], self.full.data_ptr(), self.shard_elems,
            self.world, self.rank, -1, self.copy_ctas, self.ready.data_ptr(), self.counters.data_ptr(), self.epoch,
            self.pad.data_ptr(), par * 8, self.epoch, _lib.stream_ptr())
        _lib.check_rc(rc, "gf_gemm_bf16_allgather")
        return out

    def reference(self, x_shard, w, bias=None):
        """NCCL all-gather followed by the plain GEMM kernel."""
        full = torch.empty(self.T, self.K, dtype=torch.bfloat16, device=self.device)
        dist.all_gather_into_tensor(full, x_shard.contiguous(), group=self.group)
        return gemm_raw(full, False, w, False, self.T, w.shape[0], self.K, bias=bias)


class GemmReduceScatter:
    """``out[T / world, N] = reduce_scatter(x[T, K_local] @ w[N, K_local]^T)`` in one kernel. Staging buffers and
    arrival counters are double-buffered by call parity (see :class:`AllGatherGemm` for why that suffices)."""

    def __init__(self, tokens: int, n: int, device, group=None):
        self.group = group or dist.group.WORLD
        self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        assert tokens % self.world == 0 and n % 8 == 0
        self.T, self.N = tokens, n
        self.device = torch.device(device)
        tiles_n = (n + 255) // 256
        self.ws = SymmetricWorkspace(2 * (tokens * n * 2 + tiles_n * 4 + 512) + 8192, device, self.group)
        self.stage = [self.ws.alloc(tokens * n, torch.bfloat16) for _ in range(2)]
        self.counters = [self.ws.alloc(tiles_n, torch.int32) for _ in range(2)]
        self.stage_ptrs = [_u64(self.ws.peer_ptrs(t)) for t in self.stage]
        self.counter_ptrs = [_u64(self.ws.peer_ptrs(t)) for t in self.counters]
        self.calls = 0

    def __call__(self, x: torch.Tensor, w: torch.Tensor, bias=None, residual=None, out=None):
        lib = _bind()
        Mr = self.T // self.world
        if out is None:
            out = torch.empty(Mr, self.N, dtype=torch.bfloat16, device=self.device)
        par = self.calls & 1
        rc = lib.gf_gemm_bf16_reduce_scatter(
            x.data_ptr(), w.data_ptr(), out.data_ptr(), self.T, self.N, x.shape[1], x.stride(0), w.stride(0),
            out.stride(0), bias.data_ptr() if bias is not None else None,
            residual.data_ptr() if residual is not None else None, residual.stride(0) if residual is not None else 0,
            1.0, _lib.status_word(self.device).data_ptr(), self.stage_ptrs[par], self.counter_ptrs[par], self.world,
            self.rank, self.calls >> 1, 0, _lib.stream_ptr())
        _lib.check_rc(rc, "gf_gemm_bf16_reduce_scatter")
        self.calls += 1
        return out

    def reference(self, x, w, bias=None, residual=None):
        part = gemm_raw(x, False, w, False, self.T, self.N, x.shape[1])
        out = torch.empty(self.T // self.world, self.N, dtype=torch.bfloat16, device=self.device)
        dist.reduce_scatter_tensor(out, part, group=self.group)
        if bias is not None:
            out = out + bias
        if residual is not None:
            out = out + residual
        return out


class ColumnParallelLinear(torch.nn.Module):
    """Weight ``[out / world, in]`` per rank; input token-sharded, output ``[T, out / world]``."""

    def __init__(self, in_features: int, out_features: int, tokens: int, device, group=None, fused: bool = True,
                 bias: bool = False):
        super().__init__()
        self.group = group or dist.group.WORLD
        world = dist.get_world_size(self.group)
        assert out_features % world == 0
        self.weight = torch.nn.Parameter(torch.empty(out_features // world, in_features, dtype=torch.bfloat16,
                                                     device=device).normal_(0, 0.02))
        self.bias = torch.nn.Parameter(torch.zeros(out_features // world, dtype=torch.bfloat16, device=device)) if bias else None
        self.op = AllGatherGemm(tokens, in_features, device, self.group)
        self.fused = fused

    @torch.no_grad()
    def forward(self, x_shard):
        if self.fused:
            return self.op(x_shard, self.weight, self.bias)
        return self.op.reference(x_shard, self.weight, self.bias)


class RowParallelLinear(torch.nn.Module):
    """Weight ``[out, in / world]`` per rank; input ``[T, in / world]``, output token-sharded ``[T / world, out]``."""

    def __init__(self, in_features: int, out_features: int, tokens: int, device, group=None, fused: bool = True):
        super().__init__()
        self.group = group or dist.group.WORLD
        world = dist.get_world_size(self.group)
        assert in_features % world == 0
        self.weight = torch.nn.Parameter(torch.empty(out_features, in_features // world, dtype=torch.bfloat16,
                                                     device=device).normal_(0, 0.02))
        self.op = GemmReduceScatter(tokens, out_features, device, self.group)
        self.fused = fused

    @torch.no_grad()
    def forward(self, x, residual=None):
        if self.fused:
            return self.op(x, self.weight, residual=residual)
        return self.op.reference(x, self.weight, residual=residual)
