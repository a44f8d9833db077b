"""A serving loop around one engine: callers on any thread submit requests and get futures; one worker thread owns
the engine, admits what has arrived, steps, and resolves the futures of the requests that finished. Requests that
arrive while others are decoding join the running batch at the next step (continuous batching across callers), which
a blocking ``generate`` per caller cannot give.

Reference parity: the request queue in front of the executor's step loop
(src/engine/batch_executor.rs:18-579, src/engine/executor_step.rs:859-973).
"""
from __future__ import annotations

import concurrent.futures as cf
import queue
import threading
from typing import List, Optional


class ServingLoop:
    def __init__(self, engine, idle_wait_s: float = 0.002):
        self.engine = engine
        self._inbox: "queue.Queue" = queue.Queue()
        self._futures = {}
        self._stop = threading.Event()
        self._wake = threading.Event()
        self._idle_wait = idle_wait_s
        self.stats = {"submitted": 0, "finished": 0, "steps": 0, "max_running": 0, "errors": 0}
        self._thread = threading.Thread(target=self._run, name="gllm-serving-loop", daemon=True)
        self._thread.start()

    # ---- callers --------------------------------------------------------------------------------------
    def submit(self, prompt_ids: List[int], **params) -> "cf.Future":
        """``params`` as for ``LLMEngine.add_request`` (max_tokens, temperature, top_k, top_p, eos_ids, session_id,
        stream, hook). The future resolves to the request's ``GenerateResult``; ``future.request_id`` is set once the
        engine has admitted it (None before)."""
        if self._stop.is_set():
            raise RuntimeError("the serving loop has been shut down")
        fut: cf.Future = cf.Future()
        fut.request_id = None
        self._inbox.put((list(prompt_ids), params, fut))
        self._wake.set()
        self.stats["submitted"] += 1
        return fut

    def run_in_loop(self, fn) -> "cf.Future":
        """Run ``fn()`` on the worker thread between two steps (the only thread that may touch the engine: prefix
        look-ups, page export / import for the KV distribution modes). The future resolves to its return value."""
        fut: cf.Future = cf.Future()
        self._inbox.put(("call", fn, fut))
        self._wake.set()
        return fut

    def cancel(self, fut: "cf.Future", reason: str = "aborted") -> bool:
        """Ask for a submitted request to end early (its future still resolves, with that finish reason)."""
        if fut.done():
            return False
        self._inbox.put(("cancel", fut, reason))
        self._wake.set()
        return True

    def shutdown(self, wait: bool = True):
        self._stop.set()
        self._wake.set()
        if wait:
            self._thread.join()

    # ---- the worker ------------------------------------------------------------------------------------
    def _admit(self):
        while True:
            try:
                item = self._inbox.get_nowait()
            except queue.Empty:
                return
            if item[0] == "call":
                _, fn, fut = item
                try:
                    fut.set_result(fn())
                except Exception as exc:
                    fut.set_exception(exc)
                continue
            if item[0] == "cancel":
                _, fut, reason = item
                if fut.request_id is not None:
                    self.engine.abort(fut.request_id, reason)
                else:
                    fut.cancelled_reason = reason
                continue
            prompt, params, fut = item
            if not fut.set_running_or_notify_cancel():
                continue
            if getattr(self.engine, "unhealthy", None):      # a device fault: nothing is served until the rank is reset
                fut.set_exception(RuntimeError(f"engine unhealthy: {self.engine.unhealthy}"))
                self.stats["errors"] += 1
                continue
            try:
                rid = self.engine.add_request(prompt, **params)
            except Exception as exc:          # bad request: the caller gets the error, the loop goes on
                fut.set_exception(exc)
                self.stats["errors"] += 1
                continue
            fut.request_id = rid
            self._futures[rid] = fut
            if getattr(fut, "cancelled_reason", None):
                self.engine.abort(rid, fut.cancelled_reason)

    def _run(self):
        eng = self.engine
        if getattr(eng.device, "type", "cpu") == "cuda":      # the current device is a per-thread setting
            import torch
            torch.cuda.set_device(eng.device)
        while True:
            self._admit()
            if not eng.has_work():
                if self._stop.is_set() and self._inbox.empty():
                    return
                self._wake.wait(self._idle_wait)      # sleep until something arrives (arrival order is kept)
                self._wake.clear()
                continue
            try:
                eng.step()
            except Exception as exc:          # an engine fault ends every request in flight; the loop stays usable
                for rid, fut in list(self._futures.items()):
                    if not fut.done():
                        fut.set_exception(exc)
                    self._futures.pop(rid, None)
                self.stats["errors"] += 1
                continue
            self.stats["steps"] += 1
            self.stats["max_running"] = max(self.stats["max_running"], int(eng.batcher.num_running))
            for rid in [r for r in self._futures if r in eng.results]:
                fut = self._futures.pop(rid)
                fut.set_result(eng.results.pop(rid))
                self.stats["finished"] += 1


class ReplicaRouter:
    """Data-parallel replicas of one model in one process (one engine per GPU, each behind its own ``ServingLoop``):
    a request goes to the replica whose prefix cache already holds the longest prefix of its prompt (a follow-up turn
    lands where the conversation lives), ties go to the replica with the fewest requests in flight. With
    ``fetch_on_miss`` a replica that lacks a prefix another one holds (the preferred replica is over ``max_in_flight``)
    receives the pages first (the ON_DEMAND behaviour of the KV distribution modes: export on the owner's thread, import
    on the target's, device to device). Reference: KV distribution modes of the coordinator
    (src/engine/coordinator/kv.rs:52-156, 395-569)."""

    def __init__(self, loops, fetch_on_miss: bool = True, max_in_flight: int = 1 << 30):
        self.loops = list(loops)
        self.fetch_on_miss, self.max_in_flight = fetch_on_miss, max_in_flight
        self.in_flight = [0] * len(self.loops)
        self._lock = threading.Lock()
        self.stats = {"routed": [0] * len(self.loops), "affinity_hits": 0, "fetched_pages": 0}

    def _cached_pages(self, i: int, tokens) -> int:
        full = [int(t) for t in tokens[:len(tokens) // 16 * 16]]
        if not full:
            return 0
        eng = self.loops[i].engine
        return len(self.loops[i].run_in_loop(lambda: eng.batcher.lookup_prefix_pages(full)).result())

    def submit(self, prompt_ids, **params) -> "cf.Future":
        tokens = list(prompt_ids)
        cached = [self._cached_pages(i, tokens) for i in range(len(self.loops))]
        with self._lock:
            load = list(self.in_flight)
        best = max(range(len(self.loops)), key=lambda i: (cached[i], -load[i]))
        target = best
        if load[best] >= self.max_in_flight and len(self.loops) > 1:      # the replica that has the prefix is saturated
            target = min((i for i in range(len(self.loops)) if i != best), key=lambda i: load[i])
        if cached[best] > 0 and target == best:
            self.stats["affinity_hits"] += 1
        if target != best and self.fetch_on_miss and cached[best] > cached[target]:
            src, dst = self.loops[best].engine, self.loops[target].engine
            n, pages = self.loops[best].run_in_loop(lambda: src.export_prefix_pages(tokens)).result()
            if n:
                got = self.loops[target].run_in_loop(lambda: dst.import_prefix_pages(tokens, pages)).result()
                self.stats["fetched_pages"] += got
        with self._lock:
            self.in_flight[target] += 1
        self.stats["routed"][target] += 1
        fut = self.loops[target].submit(tokens, **params)
        fut.replica = target

        def done(_):
            with self._lock:
                self.in_flight[target] -= 1
        fut.add_done_callback(done)
        return fut

    def shutdown(self):
        for lp in self.loops:
            lp.shutdown()
