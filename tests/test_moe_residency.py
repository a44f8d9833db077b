import threading
import time

import torch

from gllm_b200.moe.residency import ExpertFaultHandler, ExpertPrefetcher, PrefetchPipeline, patch_out_cold_experts


def test_fault_handler_single_loader_under_contention():
    loads = []

    def load(layer, expert):
        time.sleep(0.05)
        loads.append((layer, expert))

    h = ExpertFaultHandler(load)
    res = []
    ts = [threading.Thread(target=lambda: res.append(h.ensure(3, 7))) for _ in range(8)]
    [t.start() for t in ts]; [t.join() for t in ts]
    assert res == [True] * 8 and loads == [(3, 7)] and h.stats["waits"] == 7 and h.stats["loads"] == 1
    assert h.ensure(3, 7) and len(loads) == 1
    h.evict(3, 7); assert h.ensure(3, 7) and len(loads) == 2
    n = {"c": 0}

    def flaky(layer, expert):
        n["c"] += 1
        if n["c"] < 3:
            raise IOError("injected")
    h2 = ExpertFaultHandler(flaky, max_retries=2)
    assert h2.ensure(0, 0) and n["c"] == 3
    h3 = ExpertFaultHandler(lambda l, e: 1 / 0, max_retries=1)
    assert not h3.ensure(0, 1) and h3.stats["failures"] == 1 and isinstance(h3.errors[(0, 1)], ZeroDivisionError)


def test_prefetcher_learns_transitions_and_pipeline_accounts():
    pf = ExpertPrefetcher(num_layers=3, num_experts=8, depth=2, top=2)
    for _ in range(20):     # expert 1 at layer 0 is always followed by expert 5 at layer 1, then 2 at layer 2
        pf.observe(0, torch.tensor([[1]])); pf.observe(1, torch.tensor([[5]])); pf.observe(2, torch.tensor([[2]]))
    pred = pf.predict(0, torch.tensor([[1]]))
    assert (pred[0].layer, pred[0].expert) == (1, 5) and (pred[1].layer, pred[1].expert) == (2, 2) and pred[0].confidence > pred[1].confidence
    loaded = []
    h = ExpertFaultHandler(lambda l, e: loaded.append((l, e)))
    pipe = PrefetchPipeline(h, expert_bytes=10, max_inflight_bytes=10)
    pipe.submit(pred)
    assert pipe.pump() == 1 and loaded == [(1, 5)]
    assert pipe.pump() == 1 and loaded == [(1, 5), (2, 2)]
    assert pipe.consume(1, [5, 6]) == 1 and pipe.consume(2, [3]) == 0 and pipe.accuracy() == 0.5
    blk = torch.tensor([0, 0, 1, 2, 2, -1], dtype=torch.int32)
    assert patch_out_cold_experts(blk, [2]).tolist() == [0, 0, 1, -1, -1, -1] and patch_out_cold_experts(blk, []) is blk
