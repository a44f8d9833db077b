"""Serving metrics: latency histograms (TTFT / TPOT / ITL with p50 / p99), throughput, KV occupancy, prefix
hit rate, per-kernel roofline fractions; exported as JSON lines and, when ``prometheus_client`` is importable,
as Prometheus gauges.

Reference parity: the reference keeps structs + log lines only (``SystemState`` fields
src/scheduler/jit_types.rs:4-54; ``SequenceTelemetry`` src/scheduler/telemetry.rs:7-31); this module is the
exporter on top of the same quantities.
"""
from __future__ import annotations

import json
import math
import threading
import time
from dataclasses import dataclass, field
from typing import Dict, List, Optional


class Quantiles:
    """Exact quantiles over a bounded window (serving runs keep the last N samples)."""

    def __init__(self, window: int = 65536):
        self.window = window
        self.v: List[float] = []
        self.n = 0
        self.total = 0.0

    def add(self, x: float):
        self.n += 1
        self.total += x
        if len(self.v) >= self.window:
            self.v[self.n % self.window] = x
        else:
            self.v.append(x)

    def q(self, p: float) -> float:
        if not self.v:
            return 0.0
        s = sorted(self.v)
        return s[min(len(s) - 1, max(0, math.ceil(p * len(s)) - 1))]

    def summary(self) -> Dict[str, float]:
        return {"count": self.n, "mean": self.total / self.n if self.n else 0.0, "p50": self.q(0.5), "p90": self.q(0.9),
                "p99": self.q(0.99), "max": max(self.v) if self.v else 0.0}


@dataclass
class KernelRoofline:
    name: str
    bytes_moved: float = 0.0
    flops: float = 0.0
    seconds: float = 0.0

    def fraction(self, peak_gbs: float, peak_tflops: float) -> float:
        """Achieved / attainable for the binding resource of this kernel."""
        if self.seconds <= 0:
            return 0.0
        t_mem = self.bytes_moved / (peak_gbs * 1e9)
        t_cmp = self.flops / (peak_tflops * 1e12)
        return max(t_mem, t_cmp) / self.seconds


class MetricsRegistry:
    def __init__(self):
        self.lock = threading.Lock()
        self.hist: Dict[str, Quantiles] = {}
        self.counters: Dict[str, float] = {}
        self.gauges: Dict[str, float] = {}
        self.kernels: Dict[str, KernelRoofline] = {}
        self.t0 = time.monotonic()

    def observe(self, name: str, value: float):
        with self.lock:
            self.hist.setdefault(name, Quantiles()).add(value)

    def inc(self, name: str, n: float = 1.0):
        with self.lock:
            self.counters[name] = self.counters.get(name, 0.0) + n

    def set(self, name: str, value: float):
        with self.lock:
            self.gauges[name] = value

    def record_request(self, telemetry):
        """``telemetry``: engine.batch.SequenceTelemetry."""
        self.observe("ttft_ms", telemetry.ttft_ms)
        if telemetry.generated_tokens > 1:
            self.observe("tpot_ms", telemetry.tpot_ms)
        self.observe("e2e_ms", telemetry.e2e_ms)
        self.inc("requests")
        self.inc("prompt_tokens", telemetry.prompt_tokens)
        self.inc("generated_tokens", telemetry.generated_tokens)
        self.inc("cached_prefix_tokens", telemetry.cached_prefix_tokens)
        self.inc("preemptions", telemetry.preemptions)

    def record_kernel(self, name: str, seconds: float, bytes_moved: float = 0.0, flops: float = 0.0):
        with self.lock:
            k = self.kernels.setdefault(name, KernelRoofline(name))
            k.seconds += seconds
            k.bytes_moved += bytes_moved
            k.flops += flops

    def snapshot(self, peak_gbs: Optional[float] = None, peak_tflops: Optional[float] = None) -> dict:
        with self.lock:
            up = time.monotonic() - self.t0
            out = {"uptime_s": round(up, 3), "counters": dict(self.counters), "gauges": dict(self.gauges),
                   "histograms": {k: v.summary() for k, v in self.hist.items()}}
            gen = self.counters.get("generated_tokens", 0.0)
            out["decode_tokens_per_s"] = gen / up if up > 0 else 0.0
            pt = self.counters.get("prompt_tokens", 0.0)
            out["prefix_hit_rate"] = self.counters.get("cached_prefix_tokens", 0.0) / pt if pt else 0.0
            if peak_gbs and peak_tflops:
                out["roofline"] = {k: round(v.fraction(peak_gbs, peak_tflops), 4) for k, v in self.kernels.items()}
            return out

    def json_line(self, **kw) -> str:
        return json.dumps(self.snapshot(**kw), sort_keys=True)

    def export_prometheus(self, registry=None):
        """Mirror counters / gauges / quantiles into prometheus_client gauges (no HTTP server is started)."""
        from prometheus_client import CollectorRegistry, Gauge
        registry = registry or CollectorRegistry()
        snap = self.snapshot()
        for k, v in {**snap["counters"], **snap["gauges"]}.items():
            Gauge(f"gllm_{k}", k, registry=registry).set(v)
        for k, s in snap["histograms"].items():
            for q in ("p50", "p99"):
                Gauge(f"gllm_{k}_{q}", f"{k} {q}", registry=registry).set(s[q])
        return registry


GLOBAL = MetricsRegistry()
