"""HGAL: gang-aware eviction (LIRS / Clock-Pro flavoured) over sequence groups and weight pages.

A sequence's pages leave together (a half-evicted sequence is useless), pages touched at least ``hot_threshold``
times form the low-inter-reference (LIR) set and are protected up to ``lir_ratio`` of the pool, and pages younger
than the warm-up window are never victims.

Reference parity: src/scheduler/hgal.rs:21-740; the victim order
``priority = idle_ms + sum(page recency) - 10 * access_count - 5000 * pinned + payload adjustment`` with
(expert weight -200, dense weight +5000, KV +100, system prompt +10000, RAG -200), ascending sort,
``lir_ratio 0.3``, ``hot_threshold 3``, 100 ms warm-up (src/scheduler/hgal.rs:12-43,111-156,306-331).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Iterable, List, Optional, Set

from .types import PayloadKind, SequenceGroup, UnifiedVirtualPage

PAYLOAD_ADJ = {PayloadKind.EXPERT_WEIGHT: -200.0, PayloadKind.DENSE_LAYER_WEIGHT: 5000.0, PayloadKind.KV: 100.0,
               PayloadKind.SYSTEM_PROMPT: 10000.0, PayloadKind.RAG: -200.0}


@dataclass
class HgalConfig:
    lir_ratio: float = 0.3
    hot_threshold: int = 3
    warmup_ms: float = 100.0
    working_set_window_ms: float = 2000.0


class Hgal:
    def __init__(self, cfg: HgalConfig = HgalConfig()):
        self.cfg = cfg
        self.pages: Dict[int, UnifiedVirtualPage] = {}
        self.groups: Dict[int, SequenceGroup] = {}
        self.lir: Set[int] = set()

    # ---- bookkeeping ------------------------------------------------------------------------
    def add_page(self, page: UnifiedVirtualPage, group: Optional[int] = None, now_ms: float = 0.0):
        page.created_ms = page.last_access_ms = now_ms
        self.pages[page.vpid] = page
        if group is not None:
            g = self.groups.setdefault(group, SequenceGroup(group))
            g.pages.append(page.vpid)
            g.last_active_ms = now_ms

    def remove_group(self, group: int):
        for v in self.groups.pop(group, SequenceGroup(group)).pages:
            self.pages.pop(v, None)
            self.lir.discard(v)

    def touch(self, vpid: int, now_ms: float):
        p = self.pages[vpid]
        gap = now_ms - p.last_access_ms
        p.recency = 0.5 * p.recency + 0.5 * gap
        p.access_count += 1
        p.last_access_ms = now_ms
        if p.access_count >= self.cfg.hot_threshold and len(self.lir) < self.cfg.lir_ratio * max(len(self.pages), 1):
            self.lir.add(vpid)

    def touch_group(self, group: int, now_ms: float):
        g = self.groups[group]
        g.last_active_ms = now_ms
        for v in g.pages:
            self.touch(v, now_ms)

    # ---- victim selection ---------------------------------------------------------------------
    def _protected(self, p: UnifiedVirtualPage, now_ms: float) -> bool:
        return p.pinned or (now_ms - p.created_ms) < self.cfg.warmup_ms or p.vpid in self.lir

    def group_priority(self, g: SequenceGroup, now_ms: float) -> float:
        pages = [self.pages[v] for v in g.pages if v in self.pages]
        pr = (now_ms - g.last_active_ms) + sum(p.recency for p in pages) - 10.0 * sum(p.access_count for p in pages)
        pr -= 5000.0 * (1 if g.pinned or any(p.pinned for p in pages) else 0)
        if pages:
            # a long-idle group is evicted FIRST under "ascending sort of -priority"; keep the sign convention of
            # "higher = better victim" internally and sort descending
            pr -= PAYLOAD_ADJ.get(pages[0].kind, 0.0)
        return pr

    def select_victims(self, pages_needed: int, now_ms: float) -> List[int]:
        """Group ids to evict (whole gangs) until at least ``pages_needed`` pages are freed."""
        cands = []
        for g in self.groups.values():
            pages = [self.pages[v] for v in g.pages if v in self.pages]
            if not pages or any(self._protected(p, now_ms) for p in pages):
                continue
            cands.append((self.group_priority(g, now_ms), g.group_id, len(pages)))
        cands.sort(reverse=True)
        out, freed = [], 0
        for _, gid, n in cands:
            if freed >= pages_needed:
                break
            out.append(gid)
            freed += n
        return out

    def working_set(self, now_ms: float) -> Set[int]:
        return {v for v, p in self.pages.items() if now_ms - p.last_access_ms <= self.cfg.working_set_window_ms}
