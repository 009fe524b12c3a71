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


def zigzag_rows(seq_total: int, world: int, rank: int) -> torch.Tensor:
    """Row indices of the sequence that rank ``rank`` holds under the zig-zag assignment: the sequence is cut into
    ``2 * world`` chunks and rank r takes chunks r and 2 * world - 1 - r, so that under a causal mask every rank
    owns one early (cheap) and one late (expensive) chunk."""
    c = seq_total // (2 * world)
    lo = torch.arange(rank * c, (rank + 1) * c)
    hi = torch.arange((2 * world - 1 - rank) * c, (2 * world - rank) * c)
    return torch.cat((lo, hi))


def causal_work_per_rank(world: int, zigzag: bool) -> list[float]:
    """Share of the causal attention work (score tiles that are not masked) each rank does, for contiguous or
    zig-zag assignment; 1 / world everywhere is perfect balance. The reference only estimates such a factor for
    its single-process striped variant (ghostflow-nn/src/ring_attention.rs:333-342)."""
    n = 2 * world
    own = (lambda r: (r, n - 1 - r)) if zigzag else (lambda r: (2 * r, 2 * r + 1))
    work = [sum(a + 0.5 for a in own(r)) for r in range(world)]     # chunk a sees a full chunks and half of itself
    total = sum(work)
    return [w / total for w in work]


class ZigZagContextParallelAttention(ContextParallelAttention):
    """Causal ring attention with the zig-zag assignment of :func:`zigzag_rows`: the local rows are
    ``[early chunk ; late chunk]`` (``seq_local`` rows, one sequence per rank). With contiguous chunks the last
    rank does ``2 * world - 1`` times the work of the first and the ring runs at its pace; here every rank computes
    the same ``seq_local x seq_local / 2`` tile of scores at every ring step:

      * own K/V: early x early and late x late causal, late x early full;
      * K/V of a rank before mine: all my rows against its EARLY chunk (its late chunk lies in my future);
      * K/V of a rank after mine: my LATE rows against both of its chunks (my early rows see neither).
    """

    def __init__(self, batch, seq_local, heads, kv_heads, head_dim, group=None):
        super().__init__(batch, seq_local, heads, kv_heads, head_dim, causal=True, group=group)
        assert batch == 1 and seq_local % 2 == 0, "zig-zag is written for one sequence per rank, two chunks each"
        self.half = seq_local // 2

    def _own(self, q, k, v):
        h, H, Hkv, D = self.half, self.H, self.Hkv, self.D
        o_lo, l_lo = raw.attn_fwd(q[:h], k[:h], v[:h], 1, h, H, Hkv, D, True)
        o_hh, l_hh = raw.attn_fwd(q[h:], k[h:], v[h:], 1, h, H, Hkv, D, True)
        o_hl, l_hl = raw.attn_fwd(q[h:], k[:h], v[:h], 1, h, H, Hkv, D, False)
        o_hi, l_hi = merge_partials(o_hh, l_hh, o_hl, l_hl, 1, h, H, D)
        return torch.cat((o_lo, o_hi)), torch.cat((l_lo, l_hi), dim=2)

    def forward(self, q, k, v):
        S, h, H, Hkv, D = self.S, self.half, self.H, self.Hkv, self.D
        o, lse = self._own(q, k, v)
        if self.world == 1:
            return o, lse
        kv = torch.cat((k.reshape(-1), v.reshape(-1))).contiguous()
        nk = k.numel()
        for step in range(1, self.world):
            nxt_kv = torch.empty_like(kv)
            for w in self._exchange(kv, nxt_kv):
                w.wait()
            kv = nxt_kv
            src = (self.rank - step) % self.world
            kj, vj = kv[:nk].view_as(k), kv[nk:].view_as(v)
            if src < self.rank:
                o2, l2 = _attn_rect(q, kj[:h], vj[:h], H, Hkv, D)
                o, lse = merge_partials(o, lse, o2, l2, 1, S, H, D)
            else:
                o2, l2 = _attn_rect(q[h:], kj, vj, H, Hkv, D)
                o_hi, l_hi = merge_partials(o[h:], lse[:, :, h:], o2, l2, 1, h, H, D)
                o = torch.cat((o[:h], o_hi))
                lse = torch.cat((lse[:, :, :h], l_hi), dim=2)
        return o, lse

    def backward(self, q, k, v, o, lse, do):
        S, h, H, Hkv, D = self.S, self.half, self.H, self.Hkv, self.D
        dq = torch.zeros(q.shape, dtype=torch.float32, device=q.device)
        dk = torch.zeros(k.shape, dtype=torch.float32, device=k.device)
        dv = torch.zeros(v.shape, dtype=torch.float32, device=v.device)

        def acc(qs, ks, causal):
            """Adds the gradients of the block (query rows qs, key rows ks of the K/V at hand) in place."""
            g = _attn_rect_bwd(q[qs], kcur[ks], vcur[ks], o[qs], do[qs], lse[:, :, qs], H, Hkv, D, causal)
            dq[qs] += g[0].float()
            dkcur[ks] += g[1].float()
            dvcur[ks] += g[2].float()

        lo, hi, al = slice(0, h), slice(h, S), slice(0, S)
        kcur, vcur, dkcur, dvcur = k, v, dk, dv
        acc(lo, lo, True)
        acc(hi, hi, True)
        acc(hi, lo, False)
        if self.world == 1:
            return dq.to(q.dtype), dk.to(k.dtype), dv.to(v.dtype)
        nk = k.numel()
        pack = torch.cat((k.reshape(-1).float(), v.reshape(-1).float(), dk.reshape(-1), dv.reshape(-1))).contiguous()
        for step in range(1, self.world):
            nxt = torch.empty_like(pack)
            for w in self._exchange(pack, nxt):
                w.wait()
            pack = nxt
            src = (self.rank - step) % self.world
            kcur = pack[:nk].view_as(k).to(k.dtype)
            vcur = pack[nk:2 * nk].view_as(v).to(v.dtype)
            dkcur = pack[2 * nk:3 * nk].view(k.shape)
            dvcur = pack[3 * nk:].view(v.shape)
            if src < self.rank:
                acc(al, lo, False)
            else:
                acc(hi, al, False)
        home = torch.empty_like(pack)
        for w in self._exchange(pack, home):
            w.wait()
        return dq.to(q.dtype), home[2 * nk:3 * nk].view_as(k).to(k.dtype), home[3 * nk:].view_as(v).to(v.dtype)


def _attn_rect(q, k, v, H, Hkv, D):
    """Full (unmasked) attention of ``q [Sq, H * D]`` over ``k, v [Sk, Hkv * D]`` with Sq != Sk allowed; returns
    (o, lse [1, H, Sq]). Equal lengths go to the FlashAttention kernel, other shapes are cut into square blocks of
    the shorter length (Sq and Sk are multiples of each other here) and merged."""
    Sq, Sk = q.shape[0], k.shape[0]
    if Sq == Sk:
        return raw.attn_fwd(q, k, v, 1, Sq, H, Hkv, D, False)
    if Sq > Sk:
        parts = [raw.attn_fwd(q[i:i + Sk], k, v, 1, Sk, H, Hkv, D, False) for i in range(0, Sq, Sk)]
        return torch.cat([p[0] for p in parts]), torch.cat([p[1] for p in parts], dim=2)
    o, lse = raw.attn_fwd(q, k[:Sq], v[:Sq], 1, Sq, H, Hkv, D, False)
    for j in range(Sq, Sk, Sq):
        o2, l2 = raw.attn_fwd(q, k[j:j + Sq], v[j:j + Sq], 1, Sq, H, Hkv, D, False)
        o, lse = merge_partials(o, lse, o2, l2, 1, Sq, H, D)
    return o, lse


def _attn_rect_bwd(q, k, v, o, do, lse, H, Hkv, D, causal):
    """Gradients of one block of a larger attention whose final ``o`` / ``lse`` rows are given (so the block's
    probabilities are exp(s - lse) of the whole row). Same blocking as :func:`_attn_rect`."""
    Sq, Sk = q.shape[0], k.shape[0]
    dq, dk, dv = torch.zeros_like(q, dtype=torch.float32), torch.zeros_like(k, dtype=torch.float32), \
        torch.zeros_like(v, dtype=torch.float32)
    n = min(Sq, Sk)
    for i in range(0, Sq, n):
        for j in range(0, Sk, n):
            a, b, c = torch.empty_like(q[i:i + n]), torch.empty_like(k[j:j + n]), torch.empty_like(v[j:j + n])
            raw.attn_bwd(q[i:i + n], k[j:j + n], v[j:j + n], o[i:i + n], do[i:i + n],
                         lse[:, :, i:i + n].contiguous(), a, b, c, 1, n, H, Hkv, D, causal)
            dq[i:i + n] += a.float()
            dk[j:j + n] += b.float()
            dv[j:j + n] += c.float()
    return dq, dk, dv


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
