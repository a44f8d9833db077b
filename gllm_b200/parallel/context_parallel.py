"""Context parallelism (ring attention): the sequence is split into contiguous shards, KV blocks travel round
the ring, partial attention results are merged with an online log-sum-exp.

Reference parity: ``CpConfig{cp_size, cp_rank, pp_stage_id, sliding_window}``, contiguous shards with the
remainder spread over the first ranks (src/engine/coordinator/context_parallel.rs:76-87),
``RingAttentionPlan.execute_ring_full``: cp_size rounds of send(next) / recv(prev) of the local K/V block,
LSE merge (:286-390, 460-476), sliding-window step skipping (:103-127). The reference stages f32 on the host;
here blocks are device tensors in the KV dtype and the exchange is NCCL p2p (gloo on CPU for the tests).
Each rank lands the peer's block in its own memory before using it (no remote TMA).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import List, Optional, Tuple

import torch


@dataclass
class CpConfig:
    cp_size: int
    cp_rank: int
    pp_stage_id: int = 0
    sliding_window: int = 0


def shard_bounds(seq_len: int, cp_size: int, rank: int) -> Tuple[int, int]:
    base, rem = divmod(seq_len, cp_size)
    s = rank * base + min(rank, rem)
    return s, s + base + (1 if rank < rem else 0)


def ring_steps(cfg: CpConfig, seq_len: int, causal: bool = True) -> List[int]:
    """Source ranks whose KV block this rank needs, in ring order (own block first). Causal attention only
    looks backwards, and a sliding window drops blocks that end before the window of every local query."""
    q0, q1 = shard_bounds(seq_len, cfg.cp_size, cfg.cp_rank)
    out = []
    for step in range(cfg.cp_size):
        src = (cfg.cp_rank - step) % cfg.cp_size
        k0, k1 = shard_bounds(seq_len, cfg.cp_size, src)
        if causal and k0 >= q1:
            continue  # entirely in the future
        if cfg.sliding_window and k1 <= q0 - cfg.sliding_window + 1:
            continue  # entirely before every query's window
        out.append(src)
    return out


def partial_attention(q, k, v, q_pos, k_pos, scale, causal=True, window=0):
    """q [Tq,H,D], k/v [Tk,Hkv,D] -> (o [Tq,H,D] fp32 normalised, lse [Tq,H] natural log). Empty rows: lse=-inf."""
    H, Hkv = q.shape[1], k.shape[1]
    g = H // Hkv
    kk, vv = k.float().repeat_interleave(g, 1), v.float().repeat_interleave(g, 1)
    s = torch.einsum("qhd,khd->hqk", q.float(), kk) * scale
    mask = torch.ones(q.shape[0], k.shape[0], dtype=torch.bool, device=q.device)
    if causal:
        mask &= k_pos[None, :] <= q_pos[:, None]
    if window:
        mask &= k_pos[None, :] > q_pos[:, None] - window
    s = s.masked_fill(~mask[None], float("-inf"))
    lse = torch.logsumexp(s, -1)                                   # [H, Tq]
    p = torch.exp(s - torch.where(torch.isinf(lse), torch.zeros_like(lse), lse)[..., None])
    p = torch.where(torch.isnan(p), torch.zeros_like(p), p)
    o = torch.einsum("hqk,khd->qhd", p, vv)
    return o, lse.t().contiguous()


def merge_partials(o1, lse1, o2, lse2):
    """Online log-sum-exp merge of two normalised partial results."""
    m = torch.maximum(lse1, lse2)
    m_safe = torch.where(torch.isinf(m), torch.zeros_like(m), m)
    w1, w2 = torch.exp(lse1 - m_safe), torch.exp(lse2 - m_safe)
    den = (w1 + w2).clamp_min(1e-38)
    o = (o1 * w1[..., None] + o2 * w2[..., None]) / den[..., None]
    return o, m_safe + torch.log(den)


class RingAttention:
    def __init__(self, cfg: CpConfig, comm=None):
        self.cfg, self.comm = cfg, comm

    def run(self, q, k_local, v_local, seq_len: int, scale: Optional[float] = None, causal: bool = True):
        """q/k_local/v_local hold this rank's shard. Returns o [Tq,H,D] in q's dtype."""
        c = self.cfg
        scale = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
        q0, q1 = shard_bounds(seq_len, c.cp_size, c.cp_rank)
        q_pos = torch.arange(q0, q1, device=q.device)
        needed = set(ring_steps(c, seq_len, causal))
        o = torch.zeros(q.shape, dtype=torch.float32, device=q.device)
        lse = torch.full(q.shape[:2], float("-inf"), dtype=torch.float32, device=q.device)
        k_cur, v_cur = k_local, v_local
        nxt, prv = (c.cp_rank + 1) % c.cp_size, (c.cp_rank - 1) % c.cp_size
        for step in range(c.cp_size):
            src = (c.cp_rank - step) % c.cp_size
            if src in needed:
                k0, k1 = shard_bounds(seq_len, c.cp_size, src)
                k_pos = torch.arange(k0, k1, device=q.device)
                po, pl = partial_attention(q, k_cur, v_cur, q_pos, k_pos, scale, causal, c.sliding_window)
                o, lse = merge_partials(o, lse, po, pl)
            if step + 1 < c.cp_size and c.cp_size > 1:
                k_cur, v_cur = self._rotate(k_cur, v_cur, nxt, prv, seq_len, step)
        return o.to(q.dtype)

    def _rotate(self, k, v, nxt, prv, seq_len, step):
        """Send the block we hold to the next rank, receive the previous rank's block into local memory."""
        c = self.cfg
        src_after = (c.cp_rank - step - 1) % c.cp_size
        n0, n1 = shard_bounds(seq_len, c.cp_size, src_after)
        payload = torch.stack([k, v]).contiguous()
        incoming = torch.empty((2, n1 - n0) + tuple(k.shape[1:]), dtype=k.dtype, device=k.device)
        # even ranks send first, odd ranks receive first: no deadlock with blocking p2p
        if c.cp_rank % 2 == 0:
            self.comm.send(payload, nxt)
            self.comm.recv(incoming, prv)
        else:
            self.comm.recv(incoming, prv)
            self.comm.send(payload, nxt)
        return incoming[0], incoming[1]
