"""Observers that turn runtime counters into the ``SystemState`` the policy consumes, plus telemetry records.

Reference parity: ``BasicObserver`` -> ``SystemState`` (src/scheduler/observer.rs:55-255),
``SequenceTelemetry`` / compression telemetry (src/scheduler/telemetry.rs:7-79).
"""
from __future__ import annotations

import time
from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict

from . import SystemState


@dataclass
class CompressionTelemetry:
    pages_compressed: int = 0
    bytes_in: int = 0
    bytes_out: int = 0

    @property
    def ratio(self) -> float:
        return self.bytes_in / max(self.bytes_out, 1)


@dataclass
class StepRecord:
    t: float
    tokens: int
    prefill_tokens: int
    batch: int
    latency_ms: float


class BasicObserver:
    def __init__(self, window: int = 128):
        self.steps: Deque[StepRecord] = deque(maxlen=window)
        self.entropy_ema = 0.0
        self.sparsity_ema = 0.0
        self.compression = CompressionTelemetry()
        self.counters: Dict[str, int] = {}

    def record_step(self, tokens: int, prefill_tokens: int, batch: int, latency_ms: float):
        self.steps.append(StepRecord(time.monotonic(), tokens, prefill_tokens, batch, latency_ms))

    def record_attention(self, entropy: float, sparsity: float, alpha: float = 0.1):
        self.entropy_ema += alpha * (entropy - self.entropy_ema)
        self.sparsity_ema += alpha * (sparsity - self.sparsity_ema)

    def bump(self, name: str, n: int = 1):
        self.counters[name] = self.counters.get(name, 0) + n

    def tokens_per_second(self) -> float:
        if len(self.steps) < 2:
            return 0.0
        dt = self.steps[-1].t - self.steps[0].t
        return sum(s.tokens for s in list(self.steps)[1:]) / dt if dt > 0 else 0.0

    def system_state(self, *, free_pages: int, total_pages: int, fragmentation: float, running: int, waiting: int):
        s = SystemState()
        s.memory_pressure = 1.0 - free_pages / max(total_pages, 1)
        s.kv_fragmentation = fragmentation
        s.logits_entropy = self.entropy_ema
        s.attention_sparsity = self.sparsity_ema
        s.running = running
        s.waiting = waiting
        return s
