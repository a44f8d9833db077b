"""Weight paging: a page table over model weights (experts, dense layers) that may live in HBM, pinned host
memory or a memory-mapped file; page-fault handling with retries; per-step fault plans; a prefetch queue that can
carry a quantised copy first; a defragmenter for the device arena.

Reference parity: src/scheduler/weight_paging.rs:26-601 (page table, prefetch queue, defragmenter),
src/scheduler/fault_recovery.rs:30-794 (page-fault handler + retries, step fault plans, migration between GPUs).
Failures are injected on the host in the tests (a loader callable that raises).
"""
from __future__ import annotations

import heapq
import time
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Tuple

from .types import Tier


@dataclass
class WeightPage:
    key: str                  # e.g. "L12.experts.57"
    bytes: int
    tier: Tier = Tier.L2_CPU
    offset: int = -1          # offset in the device arena when resident
    pinned: bool = False
    last_use: int = 0
    faults: int = 0


@dataclass
class FaultPlan:
    step: int
    to_load: List[str] = field(default_factory=list)
    to_evict: List[str] = field(default_factory=list)
    stall_bytes: int = 0


class PageFaultError(RuntimeError):
    pass


class WeightPageTable:
    def __init__(self, arena_bytes: int, loader: Callable[[WeightPage, int], None], max_retries: int = 3,
                 backoff_s: float = 0.0):
        """``loader(page, offset)`` copies the page into the device arena at ``offset`` (raises on failure)."""
        self.arena_bytes, self.loader = arena_bytes, loader
        self.max_retries, self.backoff_s = max_retries, backoff_s
        self.pages: Dict[str, WeightPage] = {}
        self.free: List[Tuple[int, int]] = [(0, arena_bytes)]      # (offset, size), sorted by offset
        self.clock = 0
        self.prefetch_q: List[Tuple[float, int, str]] = []
        self._seq = 0
        self.stats = {"faults": 0, "retries": 0, "evictions": 0, "prefetched": 0, "defrag_moves": 0}

    def add(self, key: str, nbytes: int, pinned: bool = False):
        self.pages[key] = WeightPage(key, nbytes, pinned=pinned)

    # ---- arena -----------------------------------------------------------------------------------
    def _alloc(self, n: int) -> int:
        for i, (off, size) in enumerate(self.free):
            if size >= n:
                if size == n:
                    self.free.pop(i)
                else:
                    self.free[i] = (off + n, size - n)
                return off
        return -1

    def _free(self, off: int, n: int):
        self.free.append((off, n))
        self.free.sort()
        merged = []
        for o, s in self.free:
            if merged and merged[-1][0] + merged[-1][1] == o:
                merged[-1] = (merged[-1][0], merged[-1][1] + s)
            else:
                merged.append((o, s))
        self.free = merged

    def resident(self) -> List[WeightPage]:
        return [p for p in self.pages.values() if p.tier == Tier.L1_GPU]

    def fragmentation(self) -> float:
        total = sum(s for _, s in self.free)
        return 0.0 if total == 0 else 1.0 - max(s for _, s in self.free) / total

    # ---- faults ------------------------------------------------------------------------------------
    def evict(self, key: str):
        p = self.pages[key]
        if p.tier == Tier.L1_GPU and not p.pinned:
            self._free(p.offset, p.bytes)
            p.tier, p.offset = Tier.L2_CPU, -1
            self.stats["evictions"] += 1

    def ensure_resident(self, key: str) -> int:
        """Returns the arena offset; loads (evicting LRU pages if needed) with bounded retries."""
        self.clock += 1
        p = self.pages[key]
        p.last_use = self.clock
        if p.tier == Tier.L1_GPU:
            return p.offset
        self.stats["faults"] += 1
        p.faults += 1
        off = self._alloc(p.bytes)
        while off < 0:
            victims = sorted((q for q in self.resident() if not q.pinned), key=lambda q: q.last_use)
            if not victims:
                raise PageFaultError(f"no room for {key} ({p.bytes} bytes) and nothing evictable")
            self.evict(victims[0].key)
            off = self._alloc(p.bytes)
            if off < 0 and self.fragmentation() > 0.3:
                self.defragment()
                off = self._alloc(p.bytes)
        err = None
        for attempt in range(self.max_retries):
            try:
                self.loader(p, off)
                p.tier, p.offset = Tier.L1_GPU, off
                return off
            except Exception as exc:      # transient copy / IO failure: retry, then give the space back
                err = exc
                self.stats["retries"] += 1
                if self.backoff_s:
                    time.sleep(self.backoff_s * (attempt + 1))
        self._free(off, p.bytes)
        raise PageFaultError(f"loading {key} failed after {self.max_retries} attempts: {err}")

    def plan_step(self, step: int, needed: List[str]) -> FaultPlan:
        plan = FaultPlan(step)
        free = sum(s for _, s in self.free)
        missing = [k for k in needed if self.pages[k].tier != Tier.L1_GPU]
        need_bytes = sum(self.pages[k].bytes for k in missing)
        plan.to_load, plan.stall_bytes = missing, need_bytes
        if need_bytes > free:
            keep = set(needed)
            for q in sorted((q for q in self.resident() if not q.pinned and q.key not in keep), key=lambda q: q.last_use):
                if free >= need_bytes:
                    break
                plan.to_evict.append(q.key)
                free += q.bytes
        return plan

    # ---- prefetch ----------------------------------------------------------------------------------
    def enqueue_prefetch(self, key: str, priority: float):
        self._seq += 1
        heapq.heappush(self.prefetch_q, (-priority, self._seq, key))

    def run_prefetch(self, budget_bytes: int) -> List[str]:
        done = []
        while self.prefetch_q and budget_bytes > 0:
            _, _, key = heapq.heappop(self.prefetch_q)
            p = self.pages[key]
            if p.tier == Tier.L1_GPU or p.bytes > budget_bytes:
                continue
            try:
                self.ensure_resident(key)
            except PageFaultError:
                continue
            budget_bytes -= p.bytes
            self.stats["prefetched"] += 1
            done.append(key)
        return done

    # ---- defragmentation ----------------------------------------------------------------------------
    def defragment(self, mover: Optional[Callable[[WeightPage, int, int], None]] = None) -> int:
        """Slide resident pages towards offset 0. ``mover(page, old, new)`` performs the device copy."""
        moved, cursor = 0, 0
        for p in sorted(self.resident(), key=lambda q: q.offset):
            if p.offset != cursor:
                if mover:
                    mover(p, p.offset, cursor)
                p.offset = cursor
                moved += 1
            cursor += p.bytes
        self.free = [(cursor, self.arena_bytes - cursor)] if cursor < self.arena_bytes else []
        self.stats["defrag_moves"] += moved
        return moved
