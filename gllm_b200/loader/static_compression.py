"""Load-time static compression: dead-column removal in FFN weights and 2:4 structured pruning.

Reference parity: src/static_compression.rs (load-time dead-column / 2:4 pruning) and the 2:4 sparsity heuristic
of the upload path (src/loader/fragments/upload_convert.inc.rs).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Tuple

import torch


@dataclass
class DeadColumnReport:
    kept: int
    removed: int
    index: torch.Tensor


def prune_dead_ffn_columns(gate: torch.Tensor, up: torch.Tensor, down: torch.Tensor, threshold: float = 1e-6,
                           multiple_of: int = 64) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, DeadColumnReport]:
    """An intermediate neuron whose gate row, up row or down column is (near) zero contributes nothing: drop it
    from all three matrices. The kept count is rounded up to ``multiple_of`` (kernel tile granularity)."""
    alive = (gate.float().abs().amax(1) > threshold) & (up.float().abs().amax(1) > threshold) & \
            (down.float().abs().amax(0) > threshold)
    idx = torch.nonzero(alive).reshape(-1)
    pad = (-idx.numel()) % multiple_of
    if pad:
        dead = torch.nonzero(~alive).reshape(-1)[:pad]
        idx = torch.cat([idx, dead]).sort().values
    rep = DeadColumnReport(int(idx.numel()), int(gate.shape[0] - idx.numel()), idx)
    return gate[idx].contiguous(), up[idx].contiguous(), down[:, idx].contiguous(), rep


def prune_2_4(w: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Keep the two largest magnitudes of every four consecutive inputs. Returns (pruned weight, mask)."""
    n, k = w.shape
    if k % 4:
        raise ValueError("2:4 pruning needs K % 4 == 0")
    g = w.float().abs().reshape(n, k // 4, 4)
    top = g.topk(2, -1).indices
    mask = torch.zeros_like(g, dtype=torch.bool).scatter_(-1, top, True).reshape(n, k)
    return torch.where(mask, w, torch.zeros_like(w)), mask


def sparsity_2_4_fraction(w: torch.Tensor, tol: float = 0.0) -> float:
    """Fraction of 4-groups that already have at least two (near-)zeros: decides whether 2:4 storage is free."""
    g = w.float().abs().reshape(w.shape[0], -1, 4)
    return float(((g <= tol).sum(-1) >= 2).float().mean())


def pruning_error(w: torch.Tensor, pruned: torch.Tensor) -> float:
    return float((w.float() - pruned.float()).norm() / w.float().norm().clamp_min(1e-12))
