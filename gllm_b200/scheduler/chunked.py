"""Chunked-prefill sizing and interleaved batch composition rules (host-side mirrors of what the C++ batcher
applies), batch compaction and SwiftKV-style prefill distillation bookkeeping.

Reference parity: ``ChunkedConfig{min 64, max 2048, decode_slots 2}`` with the adaptive chunk by free-L1 ratio
(< 0.25 -> min, > 0.75 -> max, linear between) (src/scheduler/vllm2024.rs:15-68); ``ChunkedPrefillScheduler``
(chunk 512, decode ratio cap 0.6, max_batch_tokens 4096, compaction when the unused-slot ratio exceeds 0.25)
(src/scheduler/chunked_prefill.rs:23-330); compaction (src/scheduler/compact.rs:11-198).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Sequence, Tuple


@dataclass
class ChunkedConfig:
    min_chunk: int = 64
    max_chunk: int = 2048
    decode_slots: int = 2

    def adaptive_chunk(self, free_l1_ratio: float) -> int:
        if free_l1_ratio < 0.25:
            return self.min_chunk
        if free_l1_ratio > 0.75:
            return self.max_chunk
        f = (free_l1_ratio - 0.25) / 0.5
        return int(self.min_chunk + f * (self.max_chunk - self.min_chunk))


@dataclass
class InterleavedBatch:
    decode_ids: List[int] = field(default_factory=list)
    prefill: List[Tuple[int, int]] = field(default_factory=list)   # (request id, chunk tokens)
    budget: int = 0
    compact_required: bool = False

    @property
    def tokens(self) -> int:
        return len(self.decode_ids) + sum(c for _, c in self.prefill)


@dataclass
class ChunkedPrefillScheduler:
    chunk: int = 512
    decode_ratio_cap: float = 0.6
    max_batch_tokens: int = 4096
    compact_threshold: float = 0.25

    def compose(self, decode_ids: Sequence[int], prefill_queue: Sequence[Tuple[int, int]], memory_pressure_ratio: float = 1.0,
                slots_in_use: int = 0, slots_total: int = 0) -> InterleavedBatch:
        """Decode first (1 token each, capped at ``decode_ratio_cap`` of the budget), then prefill chunks in
        queue order until the budget is spent."""
        budget = int(self.max_batch_tokens * memory_pressure_ratio)
        b = InterleavedBatch(budget=budget)
        b.decode_ids = list(decode_ids)[: int(self.decode_ratio_cap * budget)]
        left = budget - len(b.decode_ids)
        for rid, remaining in prefill_queue:
            if left <= 0:
                break
            c = min(self.chunk, remaining, left)
            if c > 0:
                b.prefill.append((rid, c))
                left -= c
        if slots_total:
            b.compact_required = (slots_total - slots_in_use) / slots_total > self.compact_threshold and slots_in_use > 0
        return b


def compaction_plan(active_slots: Sequence[int]) -> List[Tuple[int, int]]:
    """Moves (from_slot, to_slot) that pack the active slots into [0, n) preserving their order."""
    moves = []
    for dst, src in enumerate(sorted(active_slots)):
        if src != dst:
            moves.append((src, dst))
    return moves


@dataclass
class SwiftKvPlan:
    """SwiftKV: layers past ``cut_layer`` reuse the KV projected from the cut layer's hidden state during prefill,
    so their prefill compute is skipped. This only records which layers are distilled."""
    num_layers: int
    cut_ratio: float = 0.5

    @property
    def cut_layer(self) -> int:
        return max(1, int(self.num_layers * self.cut_ratio))

    def skipped_layers(self) -> List[int]:
        return list(range(self.cut_layer, self.num_layers))

    def prefill_flop_ratio(self) -> float:
        return self.cut_layer / self.num_layers
