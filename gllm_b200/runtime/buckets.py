"""Shape bucketing driven by measurement: latency histograms, a probe that times a callable per candidate
bucket, and golden buckets that evolve with the observed length distribution.

Reference parity: micro-benchmark-driven sequence-length bucketing and runtime evolution
(src/jit/profiler.rs:187-260, src/jit/golden_bucket.rs, src/jit/histogram.rs). Here the buckets pick which CUDA
graphs (decode batch sizes) and prefill chunk lengths get captured.
"""
from __future__ import annotations

import bisect
import math
import time
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence


class LogHistogram:
    """Power-of-two-ish histogram with ``sub`` linear sub-buckets per octave (HDR style)."""

    def __init__(self, sub: int = 4, max_value: int = 1 << 20):
        self.sub = sub
        self.edges = [0]
        v = 1
        while v < max_value:
            for i in range(sub):
                e = v + (v * i) // sub
                if e > self.edges[-1]:
                    self.edges.append(e)
            v *= 2
        self.edges.append(max_value)
        self.counts = [0] * len(self.edges)
        self.total = 0

    def add(self, value: int, n: int = 1):
        i = bisect.bisect_right(self.edges, value) - 1
        self.counts[max(0, min(i, len(self.counts) - 1))] += n
        self.total += n

    def quantile(self, q: float) -> int:
        if self.total == 0:
            return 0
        need, acc = q * self.total, 0
        for i, c in enumerate(self.counts):
            acc += c
            if acc >= need:
                return self.edges[min(i + 1, len(self.edges) - 1)]
        return self.edges[-1]

    def decay(self, factor: float = 0.5):
        self.counts = [int(c * factor) for c in self.counts]
        self.total = sum(self.counts)


class LatencyProbe:
    """Times ``fn(size)`` (device-synchronised by the callable itself) for candidate sizes."""

    def __init__(self, fn: Callable[[int], None], warmup: int = 1, iters: int = 3, clock=time.perf_counter):
        self.fn, self.warmup, self.iters, self.clock = fn, warmup, iters, clock
        self.results: Dict[int, float] = {}

    def measure(self, size: int) -> float:
        for _ in range(self.warmup):
            self.fn(size)
        best = math.inf
        for _ in range(self.iters):
            t0 = self.clock()
            self.fn(size)
            best = min(best, self.clock() - t0)
        self.results[size] = best
        return best

    def knees(self, sizes: Sequence[int], tolerance: float = 0.08) -> List[int]:
        """Sizes after which latency jumps by more than ``tolerance``: natural bucket boundaries (a wave of CTAs
        filling up, a tile boundary)."""
        out, prev = [], None
        for s in sizes:
            t = self.results.get(s) or self.measure(s)
            if prev is not None and t > prev[1] * (1 + tolerance):
                out.append(prev[0])
            prev = (s, t)
        if prev:
            out.append(prev[0])
        return out


@dataclass
class GoldenBuckets:
    """A small sorted set of sizes; a request of size s runs in the smallest bucket >= s."""
    buckets: List[int] = field(default_factory=lambda: [1, 2, 4, 8, 16, 32, 64, 128, 256])
    max_buckets: int = 12
    hist: LogHistogram = field(default_factory=LogHistogram)

    def bucket_for(self, size: int) -> int:
        i = bisect.bisect_left(self.buckets, size)
        return self.buckets[i] if i < len(self.buckets) else self.buckets[-1]

    def observe(self, size: int):
        self.hist.add(size)

    def padding_waste(self) -> float:
        """Expected padded fraction under the observed distribution."""
        waste = total = 0
        for edge, c in zip(self.hist.edges, self.hist.counts):
            if c and edge > 0:
                b = self.bucket_for(edge)
                waste += c * max(0, b - edge)
                total += c * b
        return waste / total if total else 0.0

    def evolve(self, min_share: float = 0.05) -> List[int]:
        """Re-derive buckets from quantiles of the observed sizes (keeping the largest bucket as the capacity)."""
        if self.hist.total < 32:
            return self.buckets
        cap = self.buckets[-1]
        qs = sorted({max(1, self.hist.quantile(q)) for q in (0.1, 0.25, 0.5, 0.75, 0.9, 0.97, 1.0)})
        new = sorted({min(q, cap) for q in qs} | {cap})
        self.buckets = new[-self.max_buckets:]
        return self.buckets
