"""Context parallelism (ring attention): the sequence is split into contiguous shards, KV blocks travel round
the ring, partial attention results are merged with an online log-sum-exp.

Reference parity: ``CpConfig{cp_size, cp_rank, pp_stage_id, sliding_window}``, contiguous shards with the
remainder spread over the first ranks (src/engine/coordinator/context_parallel.rs:76-87),
``RingAttentionPlan.execute_ring_full``: cp_size rounds of send(next) / recv(prev) of the local K/V block,
LSE merge (:286-390, 460-476), sliding-window step skipping (:103-127). The reference stages f32 on the host;
here blocks are device tensors in the KV dtype and the exchange is NCCL p2p (gloo on CPU for the tests).
Each rank lands the peer's block in its own memory before using it (no remote TMA).

``CpPrefill`` is the form the decoder runs: a long prompt is cut into page-aligned contiguous shards, every rank runs
all layers on its shard only, and after each layer's K/V write the ranks exchange the freshly written KV pages
(one all-gather over NVSwitch: every peer is one hop away, so the blocks need not travel round a ring) and attend
with the ordinary paged prefill kernel over the pages of all earlier shards plus their own. Every rank ends with
the whole prompt's KV pages, so decoding continues on any of them.
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


class CpPrefill:
    """Context-parallel prefill of whole prompts inside ``DecoderModel.forward``.

    ``seq_lens``: prompt lengths; ``block_tables`` [S, max_blocks]: the sequences' pages in THIS rank's cache (the
    ranks may hold a logical page under different page ids: what travels is page contents, in logical order). Rank r of W owns pages [r * ceil(P / W), (r + 1) * ceil(P / W)) of a
    sequence of P pages. ``local_batch`` builds the rank's ``ForwardBatch`` (its shard's tokens at their absolute
    positions; context = everything up to the shard's end); the model calls ``exchange`` after each layer wrote its
    K/V; ``last_logits`` returns each sequence's last-token logits on every rank.
    Reference: CpConfig / RingAttentionPlan (src/engine/coordinator/context_parallel.rs:76-127, 286-390); the ring
    of send/recv rounds becomes one all-gather of pages per layer."""

    def __init__(self, cfg: CpConfig, seq_lens, block_tables: torch.Tensor, group=None, page: int = 16,
                 zigzag: bool = False):
        """``zigzag``: a sequence is cut into 2 W page-aligned chunks and rank r takes chunks r and 2 W - 1 - r, so that
        under a causal mask every rank attends over about the same number of (query, key) pairs (with contiguous
        shards the last rank does 2 W - 1 times the work of the first)."""
        self.cfg, self.group, self.page, self.zigzag = cfg, group, page, zigzag
        self.seq_lens = [int(x) for x in seq_lens]
        self.block_tables = block_tables
        W = cfg.cp_size
        n_chunks = 2 * W if zigzag else W
        self.bounds = []           # per sequence: (tok0, tok1) of chunk c
        self.chunks = []           # per sequence: per rank the list of its non-empty (tok0, tok1) chunks, ascending
        for L in self.seq_lens:
            pages = (L + page - 1) // page
            per = (pages + n_chunks - 1) // n_chunks
            cb = [(min(L, c * per * page), min(L, (c + 1) * per * page)) for c in range(n_chunks)]
            self.bounds.append(cb)
            mine = [[cb[r]] + ([cb[2 * W - 1 - r]] if zigzag else []) for r in range(W)]
            self.chunks.append([[c for c in m if c[1] > c[0]] for m in mine])
        # pages each rank writes (over all sequences), padded to one length for the all-gather
        bt = block_tables.cpu()
        self.rank_pages = []
        for r in range(W):
            ids = []
            for s in range(len(self.seq_lens)):
                for t0, t1 in self.chunks[s][r]:
                    ids += bt[s, t0 // page:(t1 + page - 1) // page].tolist()
            self.rank_pages.append(ids)
        self.max_pages = max(1, max(len(x) for x in self.rank_pages))
        dev = block_tables.device
        self._idx = [torch.tensor(ids, dtype=torch.long, device=dev) for ids in self.rank_pages]
        pad = self.rank_pages[cfg.cp_rank] + [self.rank_pages[cfg.cp_rank][-1] if self.rank_pages[cfg.cp_rank] else 0] * (
            self.max_pages - len(self.rank_pages[cfg.cp_rank]))
        self._mine_padded = torch.tensor(pad, dtype=torch.long, device=dev)
        self.owner = [next((r for r in range(W) if any(t1 == L for _, t1 in self.chunks[s][r])), 0)
                      for s, L in enumerate(self.seq_lens)]

    @staticmethod
    def every_rank_has_tokens(n_tokens: int, cp_size: int, zigzag: bool = False, page: int = 16) -> bool:
        """Whether cutting ``n_tokens`` this way leaves no rank without a token (a rank without rows cannot run)."""
        n_chunks = 2 * cp_size if zigzag else cp_size
        pages = (n_tokens + page - 1) // page
        per = (pages + n_chunks - 1) // n_chunks
        return per > 0 and (cp_size - 1) * per < pages       # chunk W - 1 (every rank's lowest chunk index is <= it)

    def local_batch(self, token_ids_per_seq):
        """The rank's prefill batch: one entry per chunk it owns (a chunk's queries are the last tokens of the context
        that ends with it); ``logits_rows`` has one row per sequence (its last token's row on the owner rank)."""
        from ..engine.batch import ForwardBatch
        r, page = self.cfg.cp_rank, self.page
        dev = self.block_tables.device
        toks, pos, slots, q_start, q_len, ctx, entry_seq = [], [], [], [], [], [], []
        rows = [0] * len(self.seq_lens)
        bt = self.block_tables.cpu()
        n = 0
        for s, ids in enumerate(token_ids_per_seq):
            for t0, t1 in self.chunks[s][r]:
                q_start.append(n)
                q_len.append(t1 - t0)
                ctx.append(t1)
                entry_seq.append(s)
                for t in range(t0, t1):
                    toks.append(int(ids[t]))
                    pos.append(t)
                    slots.append(int(bt[s, t // page]) * page + t % page)
                n += t1 - t0
                rows[s] = n - 1           # last row of the rank's highest chunk: on the owner rank the sequence's last token
        if n == 0:
            raise ValueError("context parallel prefill: this rank received no tokens (prompts shorter than one page per rank)")
        i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
        tables = self.block_tables.index_select(0, torch.tensor(entry_seq, dtype=torch.long, device=dev)).contiguous()
        b = ForwardBatch(token_ids=i32(toks), positions=i32(pos), slot_mapping=i32(slots), block_tables=tables,
                         ctx_lens=i32(ctx), q_start=i32(q_start), q_len=i32(q_len), max_q_len=max(q_len),
                         logits_rows=torch.tensor(rows, dtype=torch.long, device=dev))
        b.cp = self
        return b

    def exchange(self, kv: torch.Tensor):
        """After this rank wrote its shard's K/V into ``kv`` [pages, ...]: fetch the pages the other ranks wrote."""
        W = self.cfg.cp_size
        if W == 1:
            return
        import torch.distributed as dist
        flat = kv.view(torch.uint8).reshape(kv.shape[0], -1)      # bytes: every backend moves them
        send = flat.index_select(0, self._mine_padded)
        recv = torch.empty((W * send.shape[0], send.shape[1]), dtype=send.dtype, device=send.device)
        dist.all_gather_into_tensor(recv, send, group=self.group)
        recv = recv.view(W, send.shape[0], send.shape[1])
        for r in range(W):
            if r != self.cfg.cp_rank and len(self.rank_pages[r]):
                flat.index_copy_(0, self._idx[r], recv[r, :len(self.rank_pages[r])])

    def last_logits(self, local_logits: torch.Tensor) -> torch.Tensor:
        """[S, V] last-token logits of every sequence on every rank (from the rank that owns each last token)."""
        W = self.cfg.cp_size
        if W == 1:
            return local_logits
        import torch.distributed as dist
        S, V = local_logits.shape
        allv = torch.empty((W * S, V), dtype=local_logits.dtype, device=local_logits.device)
        dist.all_gather_into_tensor(allv, local_logits.contiguous(), group=self.group)
        allv = allv.view(W, S, V)
        return torch.stack([allv[self.owner[s], s] for s in range(len(self.seq_lens))])
