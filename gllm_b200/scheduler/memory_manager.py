"""Global memory manager: one virtual page table over the three tiers (HBM / pinned host / NVMe), session
prefix claims for multi-turn chats, pipelines, entropy-guided eviction and the prefill page plan.

Reference parity: src/scheduler/memory_manager.rs:10-860; prefill plan (all pages fit L1 -> ``FullyResident``,
else ``Pipelined{l1_pages, l2_prefetch, chunk_schedule}``): :538-580.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

from .types import KvPipeline, PayloadKind, Tier, UnifiedVirtualPage


@dataclass
class PrefillPlan:
    kind: str                               # "fully_resident" | "pipelined"
    l1_pages: int
    l2_prefetch: int = 0
    chunk_schedule: List[int] = field(default_factory=list)


@dataclass
class Session:
    session_id: str
    pages: List[int] = field(default_factory=list)
    tokens: int = 0
    finalized: bool = False
    claimed_by: Optional[int] = None


class GlobalMemoryManager:
    def __init__(self, l1_pages: int, l2_pages: int, l3_pages: int = 0, page_tokens: int = 16):
        self.cap = {Tier.L1_GPU: l1_pages, Tier.L2_CPU: l2_pages, Tier.L3_NVME: l3_pages}
        self.used = {t: 0 for t in Tier}
        self.page_tokens = page_tokens
        self.table: Dict[int, UnifiedVirtualPage] = {}
        self.sessions: Dict[str, Session] = {}
        self.entropy: Dict[int, float] = {}
        self._next = 0

    # ---- pages -------------------------------------------------------------------------------
    def free_pages(self, tier: Tier = Tier.L1_GPU) -> int:
        return self.cap[tier] - self.used[tier]

    def allocate(self, n: int, kind=PayloadKind.KV, owner=-1, pipeline=KvPipeline.CONVERSATION, tier=Tier.L1_GPU) -> List[int]:
        if self.free_pages(tier) < n:
            raise MemoryError(f"tier {tier.name}: need {n} pages, {self.free_pages(tier)} free")
        out = []
        for _ in range(n):
            v = self._next
            self._next += 1
            self.table[v] = UnifiedVirtualPage(v, kind=kind, tier=tier, owner=owner, pipeline=pipeline)
            out.append(v)
        self.used[tier] += n
        return out

    def release(self, vpids):
        for v in vpids:
            p = self.table.pop(v, None)
            if p is not None:
                self.used[p.tier] -= 1
                self.entropy.pop(v, None)

    def migrate(self, vpid: int, dst: Tier):
        p = self.table[vpid]
        if p.tier == dst:
            return
        if self.free_pages(dst) < 1:
            raise MemoryError(f"tier {dst.name} full")
        self.used[p.tier] -= 1
        self.used[dst] += 1
        p.tier = dst

    def pressure(self, tier: Tier = Tier.L1_GPU) -> float:
        return self.used[tier] / max(self.cap[tier], 1)

    # ---- sessions ------------------------------------------------------------------------------
    def claim_session(self, session_id: str, request_id: int) -> Tuple[List[int], int]:
        """Pages and token count a new turn can reuse; the session is locked to the request until finalised."""
        s = self.sessions.get(session_id)
        if s is None or not s.finalized or s.claimed_by is not None:
            return [], 0
        s.claimed_by = request_id
        return list(s.pages), s.tokens

    def finalize_session(self, session_id: str, pages: List[int], tokens: int):
        s = self.sessions.setdefault(session_id, Session(session_id))
        s.pages, s.tokens, s.finalized, s.claimed_by = list(pages), tokens, True, None
        for v in pages:
            if v in self.table:
                self.table[v].pipeline = KvPipeline.CONVERSATION

    def drop_session(self, session_id: str):
        s = self.sessions.pop(session_id, None)
        if s:
            self.release(s.pages)

    # ---- eviction ------------------------------------------------------------------------------
    def record_entropy(self, vpid: int, entropy: float):
        self.entropy[vpid] = entropy

    def entropy_victims(self, n: int) -> List[int]:
        """High-entropy pages (attention spread thin over them) carry the least information per byte: they go
        first; Working-pipeline pages before Conversation ones; pinned pages never."""
        cands = [p for p in self.table.values() if p.tier == Tier.L1_GPU and not p.pinned and p.kind == PayloadKind.KV]
        cands.sort(key=lambda p: (p.pipeline != KvPipeline.WORKING, -self.entropy.get(p.vpid, 0.0)))
        return [p.vpid for p in cands[:n]]

    # ---- prefill planning -------------------------------------------------------------------------
    def plan_prefill(self, prompt_tokens: int, chunk_tokens: int = 512) -> PrefillPlan:
        need = (prompt_tokens + self.page_tokens - 1) // self.page_tokens
        free = self.free_pages(Tier.L1_GPU)
        if need <= free:
            return PrefillPlan("fully_resident", need)
        l1 = max(free, 0)
        chunks, left = [], prompt_tokens
        while left > 0:
            c = min(chunk_tokens, left)
            chunks.append(c)
            left -= c
        return PrefillPlan("pipelined", l1, l2_prefetch=need - l1, chunk_schedule=chunks)
