"""Expert residency: fault handling for experts that are not in HBM, prefetch after the gate, the prefetch
pipeline across layers, and cold-expert patching.

Reference parity: ``ExpertFaultHandler`` thundering-herd-safe reload (src/moe/fault_handler.rs), prefetch after
the gate and its pipeline stages (src/moe/prefetch.rs, src/moe/prefetch_pipeline.rs), NOP / JMP patching of cold
experts in JIT code (src/moe/hot_patch.rs). Here "patching an expert out" means its 128-row blocks get group id
-1 in the grouped-GEMM block table, which every kernel role skips; nothing is rewritten in code memory.
"""
from __future__ import annotations

import threading
from collections import defaultdict
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence, Set

import torch


class ExpertFaultHandler:
    """Many requests may miss the same expert at once: exactly one loads it, the rest wait on its event."""

    def __init__(self, load_fn: Callable[[int, int], None], max_retries: int = 2):
        self.load_fn, self.max_retries = load_fn, max_retries
        self.resident: Set[tuple] = set()
        self.inflight: Dict[tuple, threading.Event] = {}
        self.errors: Dict[tuple, Exception] = {}
        self.lock = threading.Lock()
        self.stats = {"faults": 0, "loads": 0, "waits": 0, "failures": 0}

    def mark_resident(self, layer: int, expert: int):
        self.resident.add((layer, expert))

    def evict(self, layer: int, expert: int):
        with self.lock:
            self.resident.discard((layer, expert))

    def ensure(self, layer: int, expert: int, timeout_s: float = 30.0) -> bool:
        key = (layer, expert)
        with self.lock:
            if key in self.resident:
                return True
            self.stats["faults"] += 1
            ev = self.inflight.get(key)
            leader = ev is None
            if leader:
                ev = self.inflight[key] = threading.Event()
        if not leader:
            self.stats["waits"] += 1
            if not ev.wait(timeout_s):
                return False
            return key in self.resident
        err = None
        for _ in range(self.max_retries + 1):
            try:
                self.load_fn(layer, expert)
                err = None
                break
            except Exception as exc:
                err = exc
        with self.lock:
            if err is None:
                self.resident.add(key)
                self.stats["loads"] += 1
            else:
                self.errors[key] = err
                self.stats["failures"] += 1
            self.inflight.pop(key, None)
        ev.set()
        return err is None


@dataclass
class PrefetchRequest:
    layer: int
    expert: int
    confidence: float


class ExpertPrefetcher:
    """After layer l's gate, the chosen experts of l are needed NOW and the likely experts of l+1.. soon: a
    per-layer transition table (which experts tend to follow which) ranks the candidates."""

    def __init__(self, num_layers: int, num_experts: int, depth: int = 2, top: int = 4):
        self.L, self.E, self.depth, self.top = num_layers, num_experts, depth, top
        self.trans = [torch.zeros(num_experts, num_experts) for _ in range(num_layers)]   # [l][e_l, e_{l+1}]
        self.prev: Optional[torch.Tensor] = None

    def observe(self, layer: int, ids: torch.Tensor):
        """ids [T, k] experts chosen at ``layer``."""
        if layer > 0 and self.prev is not None and self.prev.shape[0] == ids.shape[0]:
            a = self.prev.reshape(ids.shape[0], -1, 1).long()
            b = ids.reshape(ids.shape[0], 1, -1).long()
            flat = (a * self.E + b).reshape(-1)
            self.trans[layer - 1].view(-1).index_add_(0, flat, torch.ones(flat.numel()))
        self.prev = ids.clone()

    def predict(self, layer: int, ids: torch.Tensor) -> List[PrefetchRequest]:
        out = []
        dist = torch.zeros(self.E)
        dist.index_add_(0, ids.reshape(-1).long(), torch.ones(ids.numel()))
        dist = dist / dist.sum().clamp_min(1)
        for d in range(1, self.depth + 1):
            l = layer + d
            if l >= self.L:
                break
            t = self.trans[l - 1]
            rows = t / t.sum(1, keepdim=True).clamp_min(1)
            dist = dist @ rows
            if dist.sum() <= 0:
                break
            conf, idx = dist.topk(min(self.top, self.E))
            out.extend(PrefetchRequest(l, int(e), float(c) / d) for c, e in zip(conf, idx) if c > 0)
        return sorted(out, key=lambda r: -r.confidence)


class PrefetchPipeline:
    """Stages: predicted -> issued (copy in flight on the side stream) -> ready. Bounded in-flight bytes."""

    def __init__(self, handler: ExpertFaultHandler, expert_bytes: int, max_inflight_bytes: int):
        self.handler, self.expert_bytes, self.budget = handler, expert_bytes, max_inflight_bytes
        self.predicted: List[PrefetchRequest] = []
        self.ready: Set[tuple] = set()
        self.issued = 0
        self.useful = 0

    def submit(self, reqs: Sequence[PrefetchRequest]):
        seen = {(r.layer, r.expert) for r in self.predicted}
        self.predicted.extend(r for r in reqs if (r.layer, r.expert) not in seen and (r.layer, r.expert) not in self.handler.resident)
        self.predicted.sort(key=lambda r: -r.confidence)

    def pump(self) -> int:
        n = 0
        while self.predicted and (n + 1) * self.expert_bytes <= self.budget:
            r = self.predicted.pop(0)
            if self.handler.ensure(r.layer, r.expert):
                self.ready.add((r.layer, r.expert))
                self.issued += 1
                n += 1
        return n

    def consume(self, layer: int, experts: Sequence[int]) -> int:
        hits = sum(1 for e in experts if (layer, int(e)) in self.ready)
        self.useful += hits
        return hits

    def accuracy(self) -> float:
        return self.useful / max(self.issued, 1)


def patch_out_cold_experts(blk_group: torch.Tensor, cold: Sequence[int]) -> torch.Tensor:
    """Block table with the blocks of cold experts disabled (-1): the grouped GEMMs skip them at no cost."""
    if not len(cold):
        return blk_group
    mask = torch.isin(blk_group, torch.as_tensor(list(cold), dtype=blk_group.dtype, device=blk_group.device))
    return torch.where(mask, torch.full_like(blk_group, -1), blk_group)
