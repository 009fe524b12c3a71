"""Ring attention (ghostflow-nn/src/ring_attention.rs:14-343): ``RingAttentionConfig.causal / bidirectional``,
``RingAttention.forward / max_sequence_length / memory_usage_ratio`` and ``StripedRingAttention``.

Single process: the sequence is cut into ``num_devices`` blocks and every query block visits ALL key/value
blocks in ring order with the online-softmax merge (the reference only ever visits the first
``num_devices * block_size`` keys, ring_attention.rs:133-142). Multi-process (``group`` given): each rank holds
its block of Q/K/V and the K/V blocks rotate around the ring with batched isend/irecv while the resident
block is being processed; results match attention over the whole sequence. ``StripedRingAttention``
deals tokens round-robin so that causal work is balanced across ranks.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.distributed as dist


@dataclass
class RingAttentionConfig:
    num_devices: int = 4
    block_size: int = 1024
    causal: bool = False
    overlap_comm: bool = True
    scale: float | None = None

    @classmethod
    def causal_(cls, num_devices=4, block_size=1024): return cls(num_devices, block_size, True)
    @classmethod
    def bidirectional(cls, num_devices=4, block_size=1024): return cls(num_devices, block_size, False)


RingAttentionConfig.causal_config = RingAttentionConfig.causal_


def _block_attend(q, k, v, scale, mask):
    """Partial attention of one (q block, kv block) pair -> (unnormalised out, row max, row sum)."""
    s = torch.matmul(q.float(), k.float().transpose(-1, -2)) * scale
    if mask is not None:
        s = s.masked_fill(~mask, float("-inf"))
    m = s.amax(-1)
    m_safe = torch.where(torch.isinf(m), torch.zeros_like(m), m)
    p = torch.exp(s - m_safe[..., None])
    return torch.matmul(p, v.float()), m, p.sum(-1)


def _merge(acc, m, l, o2, m2, l2):
    m_new = torch.maximum(m, m2)
    m_safe = torch.where(torch.isinf(m_new), torch.zeros_like(m_new), m_new)
    a1 = torch.exp(torch.where(torch.isinf(m), torch.full_like(m, -1e30), m) - m_safe)
    a2 = torch.exp(torch.where(torch.isinf(m2), torch.full_like(m2, -1e30), m2) - m_safe)
    return acc * a1[..., None] + o2 * a2[..., None], m_new, l * a1 + l2 * a2


class RingAttention:
    def __init__(self, config: RingAttentionConfig | None = None, group=None):
        self.config = config or RingAttentionConfig()
        self.group = group

    # positions held by ring member `r` out of `n` for a sequence of length S (contiguous blocks)
    def _positions(self, S, n, r, device):
        per = (S + n - 1) // n
        return torch.arange(r * per, min(S, (r + 1) * per), device=device)

    def forward(self, q, k, v):
        """q, k, v: ``[B, S, D]`` or ``[B, H, S, D]``. With a process group the tensors are this rank's block."""
        if self.group is not None and dist.is_initialized() and dist.get_world_size(self.group) > 1:
            return self._forward_distributed(q, k, v)
        c = self.config
        S = q.shape[-2]
        D = q.shape[-1]
        scale = c.scale if c.scale is not None else 1.0 / math.sqrt(D)
        n = max(1, min(c.num_devices, S))
        out = torch.empty_like(q, dtype=torch.float32)
        pos = [self._positions(S, n, r, q.device) for r in range(n)]
        for dq in range(n):
            pq = pos[dq]
            if pq.numel() == 0:
                continue
            qb = q.index_select(-2, pq)
            acc = torch.zeros(*qb.shape[:-1], D, device=q.device)
            m = torch.full(qb.shape[:-1], float("-inf"), device=q.device)
            l = torch.zeros(qb.shape[:-1], device=q.device)
            for step in range(n):
                dk = (dq - step) % n                 # ring order: own block first, then the left neighbour's, ...
                pk = pos[dk]
                if pk.numel() == 0:
                    continue
                mask = (pk[None, :] <= pq[:, None]) if c.causal else None
                if mask is not None and not bool(mask.any()):
                    continue
                o2, m2, l2 = _block_attend(qb, k.index_select(-2, pk), v.index_select(-2, pk), scale, mask)
                acc, m, l = _merge(acc, m, l, o2, m2, l2)
            out.index_copy_(-2, pq, acc / l.clamp(min=1e-30)[..., None])
        return out.to(q.dtype)

    def _forward_distributed(self, q, k, v):
        c = self.config
        g = self.group
        n, r = dist.get_world_size(g), dist.get_rank(g)
        Sl, D = q.shape[-2], q.shape[-1]
        scale = c.scale if c.scale is not None else 1.0 / math.sqrt(D)
        pq = self._local_positions(Sl, n, r, q.device)
        acc = torch.zeros(*q.shape[:-1], D, device=q.device)
        m = torch.full(q.shape[:-1], float("-inf"), device=q.device)
        l = torch.zeros(q.shape[:-1], device=q.device)
        kb, vb = k.contiguous(), v.contiguous()
        send_to, recv_from = (r + 1) % n, (r - 1) % n
        for step in range(n):
            src = (r - step) % n
            reqs = []
            if step + 1 < n:
                kn, vn = torch.empty_like(kb), torch.empty_like(vb)
                ops = [dist.P2POp(dist.isend, kb, send_to, g), dist.P2POp(dist.isend, vb, send_to, g),
                       dist.P2POp(dist.irecv, kn, recv_from, g), dist.P2POp(dist.irecv, vn, recv_from, g)]
                reqs = dist.batch_isend_irecv(ops)
            pk = self._local_positions(Sl, n, src, q.device)
            mask = (pk[None, :] <= pq[:, None]) if c.causal else None
            if mask is None or bool(mask.any()):
                o2, m2, l2 = _block_attend(q, kb, vb, scale, mask)
                acc, m, l = _merge(acc, m, l, o2, m2, l2)
            for rq in reqs:
                rq.wait()
            if step + 1 < n:
                kb, vb = kn, vn
        return (acc / l.clamp(min=1e-30)[..., None]).to(q.dtype)

    def _local_positions(self, Sl, n, r, device):
        return torch.arange(r * Sl, (r + 1) * Sl, device=device)

    __call__ = forward

    def max_sequence_length(self, memory_gb: float, d_model: int) -> int:
        """Longest sequence whose per-device K/V/Q blocks and one score tile fit (fp32 accounting)."""
        c = self.config
        budget = memory_gb * (1 << 30)
        per_token = 4 * d_model * 4
        tile = c.block_size * c.block_size * 4
        return int(max(0, (budget - tile) // per_token) * c.num_devices)

    def memory_usage_ratio(self, seq_len: int) -> float:
        c = self.config
        return min(1.0, (c.block_size * c.block_size) / float(max(1, seq_len) ** 2) * c.num_devices)


class StripedRingAttention(RingAttention):
    """Round-robin ("striped") token placement: member r holds tokens r, r + n, r + 2n, ... so that under a
    causal mask every ring step does a similar amount of work on every member."""

    def _positions(self, S, n, r, device):
        return torch.arange(r, S, n, device=device)

    def _local_positions(self, Sl, n, r, device):
        return torch.arange(Sl, device=device) * n + r

    def load_balance_factor(self, seq_len: int | None = None) -> float:
        """Ratio of least to most causal work among ring members (1.0 = balanced); contiguous blocks give ~1/n."""
        n = self.config.num_devices
        S = seq_len or n * self.config.block_size
        work = []
        for r in range(n):
            p = torch.arange(r, S, n)
            work.append(float((p + 1).sum()))
        return min(work) / max(work)
