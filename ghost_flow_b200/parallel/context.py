"""Context parallelism: ring attention over ranks (sequence sharded) and the Ulysses head/sequence swap.

The reference's ``RingAttention`` only does index arithmetic inside one process
(ghostflow-nn/src/ring_attention.rs:114-242 ring loop, :303-343 striped variant); here every rank holds one
contiguous chunk of the sequence, K/V chunks travel around the ring with point-to-point transfers that overlap
the FlashAttention kernel working on the chunk that has already arrived, and partial results are merged with their
log-sum-exp. The backward pass sends dK/dV around the ring together with K/V so that every chunk's gradient ends
at its owner.

Tensors use the packed layout of the attention kernels: ``q [B * S_local, Hq * D]``, ``k, v [B * S_local, Hkv * D]``.
"""
from __future__ import annotations

import math

import torch
import torch.distributed as dist

from ..ops import raw


def _world(group):
    if dist.is_available() and dist.is_initialized():
        return dist.get_world_size(group), dist.get_rank(group)
    return 1, 0


def merge_partials(o1, lse1, o2, lse2, B, S, H, D):
    """Combine two attention partials over disjoint key sets. o: [B*S, H*D]; lse: [B, H, S] (natural log)."""
    lse = torch.logaddexp(lse1, lse2)
    w1 = torch.exp(lse1 - lse).permute(0, 2, 1).reshape(B * S, H, 1)
    w2 = torch.exp(lse2 - lse).permute(0, 2, 1).reshape(B * S, H, 1)
    o = o1.float().view(B * S, H, D) * w1 + o2.float().view(B * S, H, D) * w2
    return o.view(B * S, H * D).to(o1.dtype), lse


class ContextParallelAttention:
    """Causal (or full) attention over a sequence sharded contiguously over the ranks of ``group``."""

    def __init__(self, batch, seq_local, heads, kv_heads, head_dim, causal=True, group=None):
        self.B, self.S, self.H, self.Hkv, self.D = batch, seq_local, heads, kv_heads, head_dim
        self.causal = causal
        self.group = group
        self.world, self.rank = _world(group)

    def _exchange(self, send, recv):
        """Start sending ``send`` to the next rank and receiving into ``recv`` from the previous one."""
        nxt = dist.get_global_rank(self.group, (self.rank + 1) % self.world) if self.group else (self.rank + 1) % self.world
        prv = dist.get_global_rank(self.group, (self.rank - 1) % self.world) if self.group else (self.rank - 1) % self.world
        ops = [dist.P2POp(dist.isend, send, nxt, group=self.group), dist.P2POp(dist.irecv, recv, prv, group=self.group)]
        return dist.batch_isend_irecv(ops)

    def forward(self, q, k, v):
        """Returns (o, lse); keep q, k, v, o, lse for :meth:`backward`."""
        B, S, H, Hkv, D = self.B, self.S, self.H, self.Hkv, self.D
        o, lse = raw.attn_fwd(q, k, v, B, S, H, Hkv, D, self.causal)
        if self.world == 1:
            return o, lse
        kv = torch.cat((k.reshape(-1), v.reshape(-1))).contiguous()
        nk = k.numel()
        for step in range(1, self.world):
            nxt_kv = torch.empty_like(kv)
            works = self._exchange(kv, nxt_kv)
            for w in works:
                w.wait()
            kv = nxt_kv
            src = (self.rank - step) % self.world
            if self.causal and src > self.rank:
                continue                      # that chunk lies in the future of all local queries
            kj, vj = kv[:nk].view_as(k), kv[nk:].view_as(v)
            o2, lse2 = raw.attn_fwd(q, kj, vj, B, S, H, Hkv, D, False)
            o, lse = merge_partials(o, lse, o2, lse2, B, S, H, D)
        return o, lse

    def backward(self, q, k, v, o, lse, do):
        """Returns (dq, dk, dv) for the local chunks."""
        B, S, H, Hkv, D = self.B, self.S, self.H, self.Hkv, self.D
        dq = torch.empty_like(q)
        dk, dv = torch.empty_like(k), torch.empty_like(v)
        raw.attn_bwd(q, k, v, o, do, lse, dq, dk, dv, B, S, H, Hkv, D, self.causal)
        if self.world == 1:
            return dq, dk, dv
        dq = dq.float()
        nk = k.numel()
        # the travelling packet: K, V and the gradient accumulated so far for that chunk
        pack = torch.cat((k.reshape(-1).float(), v.reshape(-1).float(), dk.reshape(-1).float(),
                          dv.reshape(-1).float())).contiguous()
        for step in range(1, self.world):
            nxt = torch.empty_like(pack)
            for w in self._exchange(pack, nxt):
                w.wait()
            pack = nxt
            src = (self.rank - step) % self.world
            if self.causal and src > self.rank:
                continue
            kj = pack[:nk].view_as(k).to(k.dtype)
            vj = pack[nk:2 * nk].view_as(v).to(v.dtype)
            dqj, dkj, dvj = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
            raw.attn_bwd(q, kj, vj, o, do, lse, dqj, dkj, dvj, B, S, H, Hkv, D, False)
            dq += dqj.float()
            pack[2 * nk:3 * nk] += dkj.reshape(-1).float()
            pack[3 * nk:] += dvj.reshape(-1).float()
        # one more hop brings every chunk's gradient home
        home = torch.empty_like(pack)
        for w in self._exchange(pack, home):
            w.wait()
        dk = home[2 * nk:3 * nk].view_as(k).to(k.dtype)
        dv = home[3 * nk:].view_as(v).to(v.dtype)
        return dq.to(q.dtype), dk, dv


class UlyssesAttention:
    """Sequence-sharded in, sequence-sharded out; inside, an all-to-all gives every rank the whole sequence for
    ``heads / world`` heads, so the local FlashAttention kernel needs no ring."""

    def __init__(self, batch, seq_local, heads, kv_heads, head_dim, causal=True, group=None):
        self.B, self.S, self.H, self.Hkv, self.D = batch, seq_local, heads, kv_heads, head_dim
        self.causal, self.group = causal, group
        self.world, self.rank = _world(group)
        assert batch == 1, "the sequence/head swap is written for one sequence per rank"
        assert heads % self.world == 0 and kv_heads % self.world == 0

    def _seq_to_heads(self, x, heads):
        """[S_local, heads * D] -> [S_local * world, heads / world * D]."""
        w, S, D = self.world, self.S, self.D
        if w == 1:
            return x
        send = x.view(S, w, heads // w * D).permute(1, 0, 2).contiguous()
        recv = torch.empty_like(send)
        dist.all_to_all_single(recv, send, group=self.group)
        return recv.view(w * S, heads // w * D)

    def _heads_to_seq(self, x, heads):
        w, S, D = self.world, self.S, self.D
        if w == 1:
            return x
        send = x.view(w, S, heads // w * D).contiguous()
        recv = torch.empty_like(send)
        dist.all_to_all_single(recv, send, group=self.group)
        return recv.permute(1, 0, 2).reshape(S, heads * D)

    def forward(self, q, k, v):
        w = self.world
        qf, kf, vf = self._seq_to_heads(q, self.H), self._seq_to_heads(k, self.Hkv), self._seq_to_heads(v, self.Hkv)
        o, lse = raw.attn_fwd(qf, kf, vf, 1, self.S * w, self.H // w, self.Hkv // w, self.D, self.causal)
        return self._heads_to_seq(o, self.H), (qf, kf, vf, o, lse)

    def backward(self, ctx, do):
        w = self.world
        qf, kf, vf, o, lse = ctx
        dof = self._seq_to_heads(do, self.H)
        dq, dk, dv = torch.empty_like(qf), torch.empty_like(kf), torch.empty_like(vf)
        raw.attn_bwd(qf, kf, vf, o, dof, lse, dq, dk, dv, 1, self.S * w, self.H // w, self.Hkv // w, self.D, self.causal)
        return self._heads_to_seq(dq, self.H), self._heads_to_seq(dk, self.Hkv), self._heads_to_seq(dv, self.Hkv)
