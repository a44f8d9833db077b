"""Epilogue telemetry: signals computed as a by-product of kernel epilogues (attention entropy, activation
sparsity, dead-neuron ratio, residual delta) aggregated into advice for gate skipping, residual bypass, sink
tracking, expert thermal state and speculation.

Reference parity: src/jit/epilogue.rs, epilogue_subsystem.rs, gate_skip.rs, residual_bypass.rs, sink_tracker.rs,
prefetch.rs; gate-skip thresholds (dead ratio > 0.5 -> CompactedCompute, > 0.3 -> MaskedCompute, else Full)
(src/engine/executor.rs:512-526).
"""
from __future__ import annotations

import enum
from collections import defaultdict
from dataclasses import dataclass, field
from typing import Dict, List, Optional

import torch


@dataclass
class EpilogueSignal:
    layer: int
    entropy: float = 0.0          # attention entropy (nats)
    sparsity: float = 0.0         # fraction of near-zero activations after the GLU
    dead_ratio: float = 0.0       # neurons that never fired in the window
    delta_rho: float = 1.0        # ||x_out - x_in|| / ||x_in||
    softmax_max: float = 0.0


def signals_from_tensors(layer: int, x_in: torch.Tensor, x_out: torch.Tensor, act: Optional[torch.Tensor] = None,
                         probs: Optional[torch.Tensor] = None, eps: float = 1e-3) -> EpilogueSignal:
    """Host-side reference of what the epilogues accumulate."""
    s = EpilogueSignal(layer)
    s.delta_rho = float((x_out.float() - x_in.float()).norm() / x_in.float().norm().clamp_min(1e-12))
    if act is not None:
        a = act.float().abs()
        s.sparsity = float((a < eps).float().mean())
        s.dead_ratio = float(((a < eps).all(0)).float().mean())
    if probs is not None:
        p = probs.float().clamp_min(1e-20)
        s.entropy = float(-(p * p.log()).sum(-1).mean())
        s.softmax_max = float(p.max(-1).values.mean())
    return s


class GateSkipMode(enum.Enum):
    FULL = "full"
    MASKED = "masked_compute"
    COMPACTED = "compacted_compute"


def gate_skip_decision(dead_ratio: float) -> GateSkipMode:
    if dead_ratio > 0.5:
        return GateSkipMode.COMPACTED
    if dead_ratio > 0.3:
        return GateSkipMode.MASKED
    return GateSkipMode.FULL


class SinkTracker:
    """Positions that keep receiving attention mass regardless of the query (attention sinks)."""

    def __init__(self, threshold: float = 0.3, min_hits: int = 4):
        self.threshold, self.min_hits = threshold, min_hits
        self.hits: Dict[int, int] = defaultdict(int)
        self.seen = 0

    def observe(self, probs: torch.Tensor):
        """probs [heads, q, k]."""
        mass = probs.float().mean((0, 1))
        for pos in torch.nonzero(mass > self.threshold).reshape(-1).tolist():
            self.hits[pos] += 1
        self.seen += 1

    def sinks(self) -> List[int]:
        return sorted(p for p, h in self.hits.items() if h >= self.min_hits)


@dataclass
class Advice:
    gate_skip: Dict[int, GateSkipMode] = field(default_factory=dict)
    bypass_layers: List[int] = field(default_factory=list)
    speculate: bool = False
    prefetch_experts: List[int] = field(default_factory=list)


class EpilogueAggregator:
    def __init__(self, num_layers: int, alpha: float = 0.2, bypass_below: float = 0.02):
        self.num_layers, self.alpha, self.bypass_below = num_layers, alpha, bypass_below
        self.ema: Dict[int, EpilogueSignal] = {}

    def push(self, s: EpilogueSignal):
        e = self.ema.get(s.layer)
        if e is None:
            self.ema[s.layer] = EpilogueSignal(**vars(s))
            return
        for f in ("entropy", "sparsity", "dead_ratio", "delta_rho", "softmax_max"):
            setattr(e, f, getattr(e, f) + self.alpha * (getattr(s, f) - getattr(e, f)))

    def advice(self) -> Advice:
        a = Advice()
        for l, e in self.ema.items():
            a.gate_skip[l] = gate_skip_decision(e.dead_ratio)
            # a layer that barely moves the residual stream can be bypassed (never the first or last two)
            if e.delta_rho < self.bypass_below and 1 < l < self.num_layers - 2:
                a.bypass_layers.append(l)
        ent = [e.entropy for e in self.ema.values()]
        a.speculate = bool(ent) and sum(ent) / len(ent) < 1.0    # confident (low-entropy) regime: drafts get accepted
        return a
