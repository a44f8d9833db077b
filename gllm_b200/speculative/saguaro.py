"""SAGUARO: speculative decoding with the draft model and the target model on different ranks.

The verify rank runs the serving engine with the target model; its drafts come from a ``RemoteDraftSource`` that
stands where the engine otherwise keeps a request's prompt-lookup index (same two calls: ``extend`` with every
committed token, ``lookup`` before a verify step). Before each verify step the source tells the draft rank which
tokens were committed since the last round (the accepted drafts plus the target's own token) and receives the next
draft; a few dozen bytes travel per round (``parallel.pd.SaguaroLink``). The draft rank (``run_draft_rank``) keeps
the committed context, proposes ``k`` greedy tokens of its small model per round, and stops on the end message.
The target's greedy choices decide what is kept, so the output equals plain greedy decoding of the target.

Reference parity: draft / verify split over two devices with token hand-off through send_bytes / recv_bytes
(src/speculative/saguaro.rs:35-490, roles :125-220).
"""
from __future__ import annotations

from typing import List, Sequence

import torch

END = -2      # length field of the message that ends a draft rank's loop


class RemoteDraftSource:
    """Draft source of ONE request on the verify rank (``engine._spec_idx[rid] = source``)."""

    def __init__(self, link, prompt: Sequence[int]):
        self.link = link
        self.pending: List[int] = []      # committed since the last round
        self.rounds = 0
        self.link.send_tokens(list(prompt), self.link.draft_rank, cap=None)      # the draft rank starts from the prompt

    def extend(self, toks: Sequence[int]):
        self.pending.extend(int(t) for t in toks)

    def lookup(self, max_len: int, top: int = 1) -> List[List[int]]:
        if not self.pending:      # nothing new since the last draft (cannot happen between two decode steps)
            return []
        self.link.send_tokens(self.pending, self.link.draft_rank)
        self.pending = []
        self.rounds += 1
        draft = self.link.recv_draft()
        return [draft[:max_len]] if draft else []

    def close(self):
        self.link.send_tokens([], self.link.draft_rank, length_field=END)


def attach_remote_drafts(engine, rid: int, link, prompt: Sequence[int]) -> RemoteDraftSource:
    """Give request ``rid`` of ``engine`` (speculative_tokens > 0) its drafts from the draft rank behind ``link``."""
    if engine.cfg.speculative_tokens <= 0:
        raise ValueError("the verify engine needs EngineConfig.speculative_tokens > 0")
    src = RemoteDraftSource(link, prompt)
    engine._spec_idx[rid] = src
    return src


def run_draft_rank(model, link, k: int) -> dict:
    """The draft rank's loop for one request: receive the prompt, then per round the committed tokens; answer with
    ``k`` greedy tokens of ``model`` continuing the committed context. Returns counters."""
    from ..engine.simple_generate import generate_single
    ctx = link.recv_tokens(link.verify_rank, cap=None)[0]
    stats = {"rounds": 0, "drafted": 0}
    while True:
        toks, length = link.recv_tokens(link.verify_rank)
        if length == END:
            return stats
        ctx = ctx + toks
        room = model.max_positions - len(ctx) - 1
        draft = generate_single(model, ctx, min(k, max(room, 0))) if room > 0 else []
        link.send_draft(draft[:link.max_draft])
        stats["rounds"] += 1
        stats["drafted"] += len(draft)
