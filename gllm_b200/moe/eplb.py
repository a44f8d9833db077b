"""Expert placement over the expert-parallel group and the load balancer that revises it.

Reference parity: ``MoeDistDecision{placement: Auto / RoundRobin (e % world) / HotCold{hot mirrored} / Custom,
all_to_all}``, ``dispatch_experts`` grouping token indices by target rank
(src/moe/distributed_dispatch.rs:19-285); EPLB: sliding-window per-expert counts, cross-rank all-reduce,
imbalance ratio (max / mean) against a threshold of 2.0, hot / cold lists -> HotCold placement
(src/moe/eplb.rs:18-243; defaults src/engine/executor_builder.rs:324-328). Counts are reduced as int64.
"""
from __future__ import annotations

import time
from collections import deque
from dataclasses import dataclass, field
from typing import Dict, List, Optional

import torch

from ..parallel.config import MoeDistConfig, MoePlacement


@dataclass
class ExpertPlacement:
    owner: List[int]                       # expert -> primary rank
    mirrors: Dict[int, List[int]] = field(default_factory=dict)   # hot expert -> extra ranks holding a copy

    def ranks_of(self, e: int) -> List[int]:
        return [self.owner[e]] + self.mirrors.get(e, [])

    def local_experts(self, rank: int) -> List[int]:
        return [e for e in range(len(self.owner)) if rank in self.ranks_of(e)]


def make_placement(cfg: MoeDistConfig, num_experts: int, world: int) -> ExpertPlacement:
    mode = cfg.placement
    if mode == MoePlacement.CUSTOM and cfg.custom_map:
        return ExpertPlacement([cfg.custom_map.get(e, e % world) for e in range(num_experts)])
    if mode == MoePlacement.ROUND_ROBIN:
        return ExpertPlacement([e % world for e in range(num_experts)])
    # Auto / HotCold: contiguous blocks (what the stacked grouped-GEMM weights want); hot experts mirrored
    per = -(-num_experts // world)
    owner = [min(e // per, world - 1) for e in range(num_experts)]
    mirrors = {}
    if mode == MoePlacement.HOT_COLD:
        for e in cfg.hot_experts:
            mirrors[e] = [r for r in range(world) if r != owner[e]]
    return ExpertPlacement(owner, mirrors)


def dispatch_experts(ids: torch.Tensor, placement: ExpertPlacement, rank: int, world: int) -> List[List[int]]:
    """(token, slot) flat indices grouped by the rank that will run them; a mirrored expert stays local when
    this rank holds a copy, else goes to its primary owner."""
    out: List[List[int]] = [[] for _ in range(world)]
    for i, e in enumerate(ids.reshape(-1).tolist()):
        ranks = placement.ranks_of(e)
        out[rank if rank in ranks else ranks[0]].append(i)
    return out


class Eplb:
    def __init__(self, num_experts: int, window_s: float = 60.0, threshold: float = 2.0, clock=time.monotonic):
        self.E, self.window_s, self.threshold, self.clock = num_experts, window_s, threshold, clock
        self.samples = deque()   # (time, counts tensor)

    def record(self, counts: torch.Tensor, now: Optional[float] = None):
        now = self.clock() if now is None else now
        self.samples.append((now, counts.to(torch.int64).cpu()))
        while self.samples and now - self.samples[0][0] > self.window_s:
            self.samples.popleft()

    def local_totals(self) -> torch.Tensor:
        t = torch.zeros(self.E, dtype=torch.int64)
        for _, c in self.samples:
            t += c
        return t

    def aggregate(self, comm=None) -> torch.Tensor:
        t = self.local_totals()
        if comm is not None and comm.world_size > 1:
            t = comm.all_reduce_counts(t)
        return t

    def imbalance(self, totals: torch.Tensor) -> float:
        mean = totals.float().mean().item()
        return float(totals.max().item() / mean) if mean > 0 else 1.0

    def decide(self, totals: torch.Tensor, cfg: MoeDistConfig) -> Optional[MoeDistConfig]:
        """New placement config when the load is imbalanced beyond the threshold, else None."""
        if self.imbalance(totals) <= self.threshold:
            return None
        mean = totals.float().mean().item()
        hot = [int(i) for i in torch.nonzero(totals.float() > self.threshold * mean).reshape(-1)]
        new = MoeDistConfig(placement=MoePlacement.HOT_COLD, all_to_all=cfg.all_to_all, hot_experts=hot,
                            eplb_window_s=cfg.eplb_window_s, eplb_threshold=cfg.eplb_threshold)
        return new
