"""Shared scheduler vocabulary.

Reference parity: src/scheduler/types.rs:4-352 (``PageState``, ``BatchOrderPolicy``, ``KvPipeline``,
``UnifiedVirtualPage`` payload kinds), src/scheduler/sequence.rs:8-77.
"""
from __future__ import annotations

import enum
from dataclasses import dataclass, field
from typing import List, Optional


class PageState(enum.IntEnum):
    FREE = 0
    ACTIVE = 1
    SHARED = 2       # bound read-only by more than one sequence (prefix reuse)
    SWAPPED = 3
    EVICTING = 4
    PINNED = 5


class BatchOrderPolicy(enum.IntEnum):
    STRICT_REQUEST_ID_ORDER = 0
    FIFO_ORDER = 1


class KvPipeline(enum.IntEnum):
    CONVERSATION = 0   # multi-turn state: never below FP8
    WORKING = 1        # scratch reasoning: may decay to nothing


class PayloadKind(enum.IntEnum):
    KV = 0
    EXPERT_WEIGHT = 1
    SYSTEM_PROMPT = 2
    RAG = 3
    DENSE_LAYER_WEIGHT = 4


class Tier(enum.IntEnum):
    L1_GPU = 0
    L2_CPU = 1
    L3_NVME = 2


@dataclass
class UnifiedVirtualPage:
    vpid: int
    kind: PayloadKind = PayloadKind.KV
    tier: Tier = Tier.L1_GPU
    physical: int = -1
    owner: int = -1                 # sequence / group id, expert id or layer id
    pinned: bool = False
    access_count: int = 0
    last_access_ms: float = 0.0
    created_ms: float = 0.0
    recency: float = 0.0
    bytes: int = 0
    pipeline: KvPipeline = KvPipeline.CONVERSATION


@dataclass
class SequenceGroup:
    group_id: int
    pages: List[int] = field(default_factory=list)
    last_active_ms: float = 0.0
    pinned: bool = False
    session: Optional[str] = None
