import pytest
import torch

from gllm_b200.runtime import (BudgetExceeded, CodeSection, CompiledVariant, ConsensusDetector, DecayingReservoir, Director,
                               DirectorSharedState, EpilogueAggregator, EpilogueSignal, GateSkipMode, GoldenBuckets, LatencyProbe,
                               LogHistogram, MechanismId, SinkTracker, VariantKey, VariantRegistry, classify, derive_constraints,
                               gate_skip_decision, host_memory_pressure, probe_system, run_ragged, signals_from_tensors, sub_batches)
from gllm_b200.runtime.sensors import CpuTopology, GpuInfo


def test_histogram_probe_and_golden_buckets():
    h = LogHistogram()
    for v in [3] * 50 + [100] * 40 + [900] * 10:
        h.add(v)
    assert h.quantile(0.5) <= 4 and 100 <= h.quantile(0.9) <= 128 and h.quantile(1.0) >= 900
    h.decay(0.5); assert h.total == 50
    fake = {1: 1.0, 2: 1.01, 4: 1.02, 8: 1.5, 16: 1.52, 32: 2.4}
    t = [0.0]
    def fn(size): t[0] += fake[size]
    p = LatencyProbe(fn, warmup=0, iters=1, clock=lambda: t[0])
    assert p.knees([1, 2, 4, 8, 16, 32]) == [4, 16, 32]
    gb = GoldenBuckets()
    assert gb.bucket_for(5) == 8 and gb.bucket_for(1000) == 256
    for s in [3] * 200 + [40] * 100 + [41] * 100:
        gb.observe(s)
    w0 = gb.padding_waste()
    new = gb.evolve()
    assert new[-1] == 256 and gb.padding_waste() <= w0 and any(40 <= b <= 48 for b in new)


def test_sub_batches_and_ragged():
    cls = classify([100, 120, 5000, 90, 100, 110, 7000], [True] * 7, "decode")
    groups = sub_batches(cls, min_size=6)
    assert sorted(len(v) for v in groups.values()) == [7]           # the short class is too small on its own: it merges up
    groups = sub_batches(cls, min_size=2)
    assert sorted(len(v) for v in groups.values()) == [2, 5]
    x = torch.arange(12.).reshape(6, 2)
    active = torch.tensor([1, 0, 1, 1, 0, 0], dtype=torch.bool)
    y = run_ragged(x.clone(), active, lambda p: p * 10)
    assert y[0].tolist() == [0., 10.] and y[1].tolist() == [2., 3.] and y[3].tolist() == [60., 70.]
    assert torch.equal(run_ragged(x.clone(), torch.zeros(6, dtype=torch.bool), lambda p: p * 0), x)


def test_epilogue_signals_gate_skip_sinks_and_advice():
    assert [gate_skip_decision(d) for d in (0.6, 0.4, 0.1)] == [GateSkipMode.COMPACTED, GateSkipMode.MASKED, GateSkipMode.FULL]
    x = torch.randn(8, 16)
    act = torch.randn(8, 32); act[:, :20] = 0
    probs = torch.softmax(torch.randn(2, 8, 8) * 5, -1)
    s = signals_from_tensors(3, x, x * 1.01, act, probs)
    assert abs(s.delta_rho - 0.01) < 1e-4 and abs(s.dead_ratio - 20 / 32) < 1e-6 and 0 < s.entropy < 2.08
    agg = EpilogueAggregator(num_layers=8)
    for l in range(8):
        agg.push(EpilogueSignal(l, entropy=0.5, dead_ratio=0.6 if l == 4 else 0.0, delta_rho=0.001 if l in (0, 3, 7) else 0.5))
    a = agg.advice()
    assert a.gate_skip[4] == GateSkipMode.COMPACTED and a.bypass_layers == [3] and a.speculate
    st = SinkTracker(threshold=0.3, min_hits=2)
    p = torch.zeros(2, 4, 6); p[..., 0] = 0.6; p[..., 5] = 0.4
    st.observe(p); st.observe(p)
    assert st.sinks() == [0, 5]


def test_variant_registry_budget_and_selection():
    r = VariantRegistry(budget_bytes=1000)
    for b in (8, 32, 128):
        r.register(CompiledVariant(VariantKey(b), handle=f"g{b}", bytes=200))
    assert r.select_for_batch(20).handle == "g32" and r.select_for_batch(500) is None
    assert r.select_for_batch(4, (MechanismId.DENSE, MechanismId.SAMPLED)) is None
    r.register(CompiledVariant(VariantKey(256), handle="g256", bytes=300))       # evicts a never-hit variant
    assert r.used() <= 800 and VariantKey(32) in r.variants
    with pytest.raises(BudgetExceeded):
        r.register(CompiledVariant(VariantKey(512), handle="x", bytes=900), evict=False)
    for _ in range(50):
        r.select_for_batch(20)
    r.reclassify()
    assert r.variants[VariantKey(32)].section == CodeSection.HOT


def test_director_consensus_and_reservoir():
    res = DecayingReservoir(capacity=8)
    for i in range(100):
        res.add(float(i))
    assert len(res.items) == 8 and res.quantile(0.5) >= 0
    det = ConsensusDetector(quorum=2)
    assert det.observe("k", 1, True) is None and det.observe("k", 1, True) is not None and det.observe("k", 1, True) is None
    assert det.observe("k", 1, False) is None and det.observe("k", 1, True) is None
    st = DirectorSharedState(expert_hits={0: 5, 1: 0}, head_mass={3: 0.0})
    got = []
    d = Director(st, on_event=got.append, quorum=2)
    d.poll_once(now=1.0)
    st.expert_hits[0] = 3
    ev = d.poll_once(now=2.0)
    assert {(e.kind, e.subject) for e in ev} == {("cold_expert", 1), ("attention_silence", 3)} and len(got) == 2
    d.interval_s = 0.01; d.spawn(); d.stop()


def test_sensors():
    assert 0.0 <= host_memory_pressure() <= 1.0
    assert host_memory_pressure({"MemTotal": 100, "MemAvailable": 25}) == 0.75
    topo = probe_system()
    assert topo.cpu.logical_cores >= 1 and topo.numa.nodes >= 1
    c = derive_constraints(CpuTopology(flags=["avx2"]), GpuInfo(present=True, sm_count=148, cc_major=10, l2_bytes=126 << 20), 0.25)
    assert c.simd_width_bits == 256 and (c.tile_m, c.tile_n) == (128, 256) and c.sm_partition.comm_sms == 37
