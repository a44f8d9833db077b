"""Tracing: NVTX ranges (visible to Nsight tools), CUDA-event device timers, and a Chrome-trace writer.

Device timing follows one rule: events recorded on the launching stream, read after a synchronise; multi-GPU
numbers are the maximum over ranks.
"""
from __future__ import annotations

import contextlib
import json
import os
import threading
import time
from typing import Dict, List, Optional

import torch

_enabled = os.environ.get("GLLM_TRACE", "0") == "1"


def enable(on: bool = True):
    global _enabled
    _enabled = on


@contextlib.contextmanager
def nvtx_range(name: str):
    """NVTX range when CUDA is present and tracing is on; free otherwise."""
    use = _enabled and torch.cuda.is_available()
    if use:
        torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        if use:
            torch.cuda.nvtx.range_pop()


class DeviceTimer:
    """Accumulates CUDA-event intervals by name; ``results`` synchronises once and returns milliseconds."""

    def __init__(self):
        self.pending: List[tuple] = []
        self.ms: Dict[str, float] = {}
        self.calls: Dict[str, int] = {}

    @contextlib.contextmanager
    def section(self, name: str):
        if not torch.cuda.is_available():
            t0 = time.perf_counter()
            yield
            self.ms[name] = self.ms.get(name, 0.0) + (time.perf_counter() - t0) * 1e3
            self.calls[name] = self.calls.get(name, 0) + 1
            return
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        yield
        b.record()
        self.pending.append((name, a, b))

    def results(self) -> Dict[str, float]:
        if self.pending:
            torch.cuda.synchronize()
            for name, a, b in self.pending:
                self.ms[name] = self.ms.get(name, 0.0) + a.elapsed_time(b)
                self.calls[name] = self.calls.get(name, 0) + 1
            self.pending = []
        return dict(self.ms)

    def max_over_ranks(self, group=None) -> Dict[str, float]:
        res = self.results()
        import torch.distributed as dist
        if not (dist.is_available() and dist.is_initialized()):
            return res
        names = sorted(res)
        dev = "cuda" if torch.cuda.is_available() and dist.get_backend(group) == "nccl" else "cpu"
        t = torch.tensor([res[n] for n in names], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
        return dict(zip(names, t.tolist()))


class GraphTimer:
    """Per-op device time of a step that runs as a CUDA graph. ``mark(name)`` after an op records an event (an
    external event-record node when called during stream capture); ``results`` attributes the interval since the
    previous mark of the same capture to ``name``. Marks whose events did not fire in the last replay are skipped."""

    def __init__(self, eager: bool = False):
        self.marks: List[tuple] = []
        self.eager = eager      # also time eagerly launched steps (prefill chunks)

    def mark(self, name: str):
        if not torch.cuda.is_available():
            return
        capturing = torch.cuda.is_current_stream_capturing()
        if not capturing and not self.eager:
            return      # only the captured step is timed, not its eager warm-up
        e = torch.cuda.Event(enable_timing=True, external=capturing)
        e.record()
        self.marks.append((name, e))

    def results(self) -> Dict[str, float]:
        if not self.marks:
            return {}
        torch.cuda.synchronize()
        out: Dict[str, float] = {}
        prev = None
        for name, e in self.marks:
            if name == "begin" or prev is None:
                prev = e
                continue
            try:
                dt = prev.elapsed_time(e)
            except Exception:      # not part of the last replayed graph
                prev = e
                continue
            if dt >= 0:
                out[name] = out.get(name, 0.0) + dt
            prev = e
        return out


class ChromeTrace:
    """Host-side spans in the Chrome / Perfetto trace-event format."""

    def __init__(self):
        self.events: List[dict] = []
        self.lock = threading.Lock()
        self.t0 = time.perf_counter()

    @contextlib.contextmanager
    def span(self, name: str, cat: str = "engine", **args):
        s = (time.perf_counter() - self.t0) * 1e6
        try:
            yield
        finally:
            e = (time.perf_counter() - self.t0) * 1e6
            with self.lock:
                self.events.append({"name": name, "cat": cat, "ph": "X", "ts": s, "dur": e - s, "pid": os.getpid(),
                                    "tid": threading.get_ident() % 100000, "args": args})

    def counter(self, name: str, **values):
        with self.lock:
            self.events.append({"name": name, "ph": "C", "ts": (time.perf_counter() - self.t0) * 1e6, "pid": os.getpid(),
                                "args": values})

    def save(self, path: str):
        with open(path, "w") as f:
            json.dump({"traceEvents": self.events, "displayTimeUnit": "ms"}, f)
