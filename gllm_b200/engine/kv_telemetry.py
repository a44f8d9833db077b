"""Attention telemetry of the KV pages, the 64-byte page headers it lands in, and the importance scores the KV
optimiser derives from it.

The reference's attention epilogue writes, per KV page, how the newest query looked at it (entropy of the attention
inside the page, the largest probability, how differently the heads weigh it) into the page header; the scheduler's KV
optimiser turns that into an importance score and a precision tier per page (src/jit/epilogue.rs; header fields
src/kv_cache/mod.rs:119-135; score and tiers src/scheduler/kv_optimizer.rs:55-192). Here the same quantities are
sampled after a decode step from what the step left behind: the last layer's post-RoPE queries in the model's
workspace and that layer's cache pages. It is a sampled, eager pass (a few tensor ops per running sequence), not part
of the captured step: ``EngineConfig.kv_telemetry_every`` sets how often it runs (0 = never).

Per request the result feeds ``LLMEngine.kv_importance`` (the largest page score, so that one sink-like page keeps
the request at full precision), which decides the tier a preempted request may wait in (``LLMEngine._swap_tier``).
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

from ..kv_cache.header import KvPageHeaderTable
from ..scheduler.kv_optimizer import decide_tier, importance_score, is_sink_page


def attention_page_stats(q_row: torch.Tensor, kv_layer: torch.Tensor, pages: List[int], ctx: int, n_q: int, n_kv: int,
                         scale: float, kv_scale: float = 1.0) -> Dict[str, torch.Tensor]:
    """How one query row attends over a sequence's pages in one layer.

    q_row [n_q * D]; kv_layer [num_pages, 2, n_kv, 16, D]; ``pages``: the sequence's block table (first ceil(ctx / 16)
    entries used). Returns per page (mean over heads unless said otherwise): ``mass`` (attention probability that
    falls into the page), ``entropy`` (nats, of the attention renormalised inside the page), ``softmax_max`` (largest
    single probability in the page, max over heads), ``head_spread`` (0..255: spread of the heads' masses), and the
    attention output ``out`` [n_q, D] of the row (for checking the alignment with the step's own attention)."""
    D = kv_layer.shape[-1]
    n_pages = (ctx + 15) // 16
    idx = torch.as_tensor(pages[:n_pages], dtype=torch.long, device=kv_layer.device)
    blk = kv_layer.index_select(0, idx)                                       # [P, 2, n_kv, 16, D]
    blk = blk.float() * kv_scale if blk.dtype == torch.float8_e4m3fn else blk.float()
    g = n_q // n_kv
    k = blk[:, 0].permute(1, 0, 2, 3).reshape(n_kv, n_pages * 16, D)[:, :ctx]           # [n_kv, ctx, D]
    v = blk[:, 1].permute(1, 0, 2, 3).reshape(n_kv, n_pages * 16, D)[:, :ctx]
    q = q_row.float().reshape(n_kv, g, D)
    s = torch.einsum("hgd,htd->hgt", q, k) * scale                             # [n_kv, g, ctx]
    p = torch.softmax(s, -1)
    out = torch.einsum("hgt,htd->hgd", p, v).reshape(n_q, D)
    pad = n_pages * 16 - ctx
    pp = torch.nn.functional.pad(p, (0, pad)).reshape(n_q, n_pages, 16)        # [heads, P, 16]
    mass_h = pp.sum(-1)                                                        # [heads, P]
    inner = pp / mass_h.clamp_min(1e-20)[..., None]
    ent = -(inner * torch.log(inner.clamp_min(1e-20))).sum(-1)                 # [heads, P]
    return {"mass": mass_h.mean(0), "entropy": ent.mean(0), "softmax_max": pp.amax(-1).amax(0),
            "head_spread": (mass_h.std(0, unbiased=False) / mass_h.mean(0).clamp_min(1e-12)).clamp(0, 1).mul(255).round(),
            "out": out}


class KvTelemetry:
    """Page headers of an engine's pool, filled by sampling the running sequences after a decode step."""

    def __init__(self, engine):
        self.engine = engine
        self.headers = KvPageHeaderTable(engine.num_pages)
        self.samples = 0

    def sample(self, plan, max_sequences: Optional[int] = None) -> Dict[int, int]:
        """One pass over the sequences of the decode step that just ran (``plan``: the step's plan; the workspace rows
        are slot-indexed like the plan's arrays); returns {request: importance 0..255} and stores it in
        ``engine.kv_importance``. Page entropy is scaled to the score's range (a page holds 16 tokens: ln 16 nats at
        most, the score formula expects up to ln 1024 = 6.93 for a context-wide distribution)."""
        eng = self.engine
        model = eng.model
        ws = getattr(model, "_ws", None)
        if ws is None or model.cfg.is_mla or getattr(model.cfg, "gemma3n_structure", False):
            return {}
        layer = len(model.layers) - 1
        if model.layers[layer].kv_donor is not None:
            return {}            # the workspace holds the LAST layer's queries and that layer has no pages of its own
        kv = eng.kv_caches[layer]
        out: Dict[int, int] = {}
        slots = [int(sl) for sl in (plan.dec_seq_ids >= 0).nonzero()[0]]
        if max_sequences is not None and len(slots) > max_sequences:      # a rotating window over the running set
            start = (self.samples * max_sequences) % len(slots)
            slots = (slots + slots)[start:start + max_sequences]
        for slot in slots:
            rid, ctx = int(plan.dec_seq_ids[slot]), int(plan.dec_positions[slot]) + 1
            pages = list(eng.batcher.block_table_of(rid))
            if ctx < 1 or len(pages) * 16 < ctx:
                continue
            stats = attention_page_stats(ws.q[slot], kv, pages, ctx, model.n_q_local, model.n_kv_local, model.scale,
                                         model.kv_scale)
            self.last_out = {"request": rid, "slot": slot, "out": stats["out"]}
            best = 0
            n_pages = (ctx + 15) // 16
            for j in range(n_pages):
                ent = float(stats["entropy"][j]) * (6.93 / math.log(16.0))
                smax, spread = float(stats["softmax_max"][j]), int(stats["head_spread"][j])
                score = importance_score(ent, smax, spread, 1.0)
                sink = is_sink_page(score, has_sink_token=(j == 0))
                page = pages[j]
                if int(self.headers.h["sequence_id"][page]) != rid or int(self.headers.h["ref_count"][page]) == 0:
                    self.headers.bind(page, rid, j, now=eng._steps, pipeline=0 if rid in eng._sessions else 1)
                self.headers.record_telemetry(page, ent, smax, 1.0, head_spread=spread, centroid=float(stats["mass"][j]))
                self.headers.h["importance"][page] = score
                self.headers.h["precision_tier"][page] = int(decide_tier(score, sink=sink))
                if not (j == 0 and n_pages > 1):       # the sink page is kept apart anyway
                    best = max(best, score)
            out[rid] = best
            eng.kv_importance[rid] = best
        self.samples += 1
        return out
