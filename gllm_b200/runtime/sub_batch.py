"""Sub-batch dispatch by shape class and ragged compaction of the active lanes.

Reference parity: shape-class sub-batches (src/jit/sub_batch.rs) and compact -> execute -> scatter of active
lanes (src/jit/ragged.rs).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, List, Sequence, Tuple

import torch


@dataclass(frozen=True)
class ShapeClass:
    ctx_bucket: int       # context length bucket (pages)
    greedy: bool
    phase: str            # "decode" | "prefill"


def classify(ctx_lens: Sequence[int], greedy: Sequence[bool], phase: str, ctx_edges=(256, 1024, 4096, 16384)) -> List[ShapeClass]:
    out = []
    for c, g in zip(ctx_lens, greedy):
        b = next((e for e in ctx_edges if c <= e), ctx_edges[-1] * 4)
        out.append(ShapeClass(b, bool(g), phase))
    return out


def sub_batches(classes: Sequence[ShapeClass], min_size: int = 4) -> Dict[ShapeClass, List[int]]:
    """Lane indices per shape class; classes smaller than ``min_size`` are merged into the next larger context
    bucket of the same kind (a launch per tiny class costs more than the padding)."""
    groups: Dict[ShapeClass, List[int]] = {}
    for i, c in enumerate(classes):
        groups.setdefault(c, []).append(i)
    keys = sorted(groups, key=lambda k: (k.phase, k.greedy, k.ctx_bucket))
    for k in keys:
        if k in groups and len(groups[k]) < min_size:
            bigger = [j for j in groups if j != k and j.phase == k.phase and j.greedy == k.greedy and j.ctx_bucket > k.ctx_bucket]
            if bigger:
                tgt = min(bigger, key=lambda j: j.ctx_bucket)
                groups[tgt] = sorted(groups[tgt] + groups.pop(k))
    return groups


def compact(x: torch.Tensor, active: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Gather the active rows to the front. Returns (packed rows, their original indices)."""
    idx = torch.nonzero(active, as_tuple=False).reshape(-1)
    return x.index_select(0, idx), idx


def scatter_back(full: torch.Tensor, packed: torch.Tensor, idx: torch.Tensor) -> torch.Tensor:
    full.index_copy_(0, idx, packed)
    return full


def run_ragged(x: torch.Tensor, active: torch.Tensor, fn: Callable[[torch.Tensor], torch.Tensor]) -> torch.Tensor:
    """compact -> execute -> scatter: inactive lanes keep their old values."""
    packed, idx = compact(x, active)
    if packed.shape[0] == 0:
        return x
    return scatter_back(x, fn(packed), idx)
