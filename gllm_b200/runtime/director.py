"""Background director: watches decayed statistics and raises consensus events (an expert nobody routes to, an
attention head that went silent, a bucket distribution that drifted) that trigger re-planning off the hot path.

Reference parity: ``DecayingReservoir`` (src/jit/director.rs:29), ``ConsensusDetector`` / ``ConsensusEvent``
(:97-119), ``DirectorSharedState`` (:218), ``JitDirector::spawn`` (:317-330).
"""
from __future__ import annotations

import random
import threading
import time
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional


class DecayingReservoir:
    """Reservoir sample whose old entries are displaced with a bias towards recency."""

    def __init__(self, capacity: int = 256, decay: float = 0.98, seed: int = 0):
        self.capacity, self.decay = capacity, decay
        self.items: List[float] = []
        self.weight = 0.0
        self.rng = random.Random(seed)

    def add(self, x: float):
        self.weight = self.weight * self.decay + 1.0
        if len(self.items) < self.capacity:
            self.items.append(x)
        elif self.rng.random() < self.capacity / max(self.weight, self.capacity):
            self.items[self.rng.randrange(self.capacity)] = x

    def mean(self) -> float:
        return sum(self.items) / len(self.items) if self.items else 0.0

    def quantile(self, q: float) -> float:
        if not self.items:
            return 0.0
        s = sorted(self.items)
        return s[min(len(s) - 1, int(q * len(s)))]


@dataclass
class ConsensusEvent:
    kind: str            # "cold_expert" | "attention_silence" | "bucket_drift"
    subject: int
    evidence: float
    at: float = 0.0


class ConsensusDetector:
    """An event fires only after ``quorum`` consecutive observation windows agree."""

    def __init__(self, quorum: int = 3):
        self.quorum = quorum
        self.streak: Dict[tuple, int] = {}

    def observe(self, kind: str, subject: int, condition: bool, evidence: float = 0.0, now: float = 0.0) -> Optional[ConsensusEvent]:
        k = (kind, subject)
        if not condition:
            self.streak.pop(k, None)
            return None
        self.streak[k] = self.streak.get(k, 0) + 1
        if self.streak[k] == self.quorum:
            return ConsensusEvent(kind, subject, evidence, now)
        return None


@dataclass
class DirectorSharedState:
    expert_hits: Dict[int, int] = field(default_factory=dict)
    head_mass: Dict[int, float] = field(default_factory=dict)
    batch_sizes: DecayingReservoir = field(default_factory=DecayingReservoir)
    events: List[ConsensusEvent] = field(default_factory=list)
    lock: threading.Lock = field(default_factory=threading.Lock)


class Director:
    def __init__(self, state: DirectorSharedState, on_event: Optional[Callable[[ConsensusEvent], None]] = None,
                 interval_s: float = 1.0, quorum: int = 3):
        self.state, self.on_event, self.interval_s = state, on_event, interval_s
        self.detector = ConsensusDetector(quorum)
        self._halt = threading.Event()
        self._thread: Optional[threading.Thread] = None
        self._last_bucket_mean: Optional[float] = None

    def poll_once(self, now: Optional[float] = None) -> List[ConsensusEvent]:
        now = time.monotonic() if now is None else now
        fired = []
        with self.state.lock:
            hits, heads = dict(self.state.expert_hits), dict(self.state.head_mass)
            for e in self.state.expert_hits:
                self.state.expert_hits[e] = 0
            mean_b = self.state.batch_sizes.mean()
        for e, h in hits.items():
            ev = self.detector.observe("cold_expert", e, h == 0, 0.0, now)
            if ev:
                fired.append(ev)
        for h, m in heads.items():
            ev = self.detector.observe("attention_silence", h, m < 1e-3, m, now)
            if ev:
                fired.append(ev)
        if self._last_bucket_mean is not None and self._last_bucket_mean > 0:
            drift = abs(mean_b - self._last_bucket_mean) / self._last_bucket_mean
            ev = self.detector.observe("bucket_drift", 0, drift > 0.5, drift, now)
            if ev:
                fired.append(ev)
                self._last_bucket_mean = mean_b
        else:
            self._last_bucket_mean = mean_b
        with self.state.lock:
            self.state.events.extend(fired)
        for ev in fired:
            if self.on_event:
                self.on_event(ev)
        return fired

    def spawn(self):
        def loop():
            while not self._halt.wait(self.interval_s):
                self.poll_once()
        self._thread = threading.Thread(target=loop, name="gllm-director", daemon=True)
        self._thread.start()
        return self

    def stop(self):
        self._halt.set()
        if self._thread:
            self._thread.join(timeout=2)
