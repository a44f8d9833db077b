import os

import pytest
import torch

from gllm_b200.kv_cache.header import CompressionCodec, PrecisionTier, StorageTier
from gllm_b200.scheduler.chunked import ChunkedConfig, ChunkedPrefillScheduler, SwiftKvPlan, compaction_plan
from gllm_b200.scheduler.hgal import Hgal, HgalConfig
from gllm_b200.scheduler.kv_optimizer import decide_tier, importance_score, is_sink_page, requantize_page
from gllm_b200.scheduler.memory_manager import GlobalMemoryManager
from gllm_b200.scheduler.observer import BasicObserver
from gllm_b200.scheduler.request_state import ExitFlag, Phase, RequestStateTable
from gllm_b200.scheduler.swap import (BackgroundWorker, DmaCommand, NvmeSwapFile, ThreeTierSwap, compress, crc16_ccitt,
                                      decompress, rle_bitpack_decode, rle_bitpack_encode)
from gllm_b200.scheduler.types import KvPipeline, PayloadKind, Tier, UnifiedVirtualPage
from gllm_b200.scheduler.weight_paging import PageFaultError, WeightPageTable


def test_hgal_gang_eviction_order_and_protection():
    h = Hgal(HgalConfig(warmup_ms=100))
    for g, kind in ((1, PayloadKind.KV), (2, PayloadKind.KV), (3, PayloadKind.SYSTEM_PROMPT), (4, PayloadKind.EXPERT_WEIGHT)):
        for i in range(3):
            h.add_page(UnifiedVirtualPage(g * 10 + i, kind=kind), group=g, now_ms=0)
    for _ in range(4):
        h.touch(11, 850)                                       # one hot page makes group 1 LIR-protected
    assert 11 in h.lir
    h.touch_group(2, 900); h.touch_group(2, 950)               # group 2 is in recent use
    v = h.select_victims(3, now_ms=1000)
    assert v == [4]                                            # expert weights go first; system prompt last
    v = h.select_victims(6, now_ms=1000)
    assert v[0] == 4 and 1 not in v and v[-1] in (2, 3) and v[1] == 2
    h.add_page(UnifiedVirtualPage(99), group=9, now_ms=990)
    assert 9 not in h.select_victims(100, now_ms=1000)         # warm-up protection
    assert 99 in h.working_set(1000) and 40 not in h.working_set(5000)
    h.remove_group(4)
    assert 40 not in h.pages


def test_memory_manager_tiers_sessions_and_prefill_plan():
    mm = GlobalMemoryManager(l1_pages=8, l2_pages=16, l3_pages=4)
    a = mm.allocate(6, owner=1)
    assert mm.free_pages() == 2 and abs(mm.pressure() - 0.75) < 1e-9
    assert mm.plan_prefill(32).kind == "fully_resident"
    plan = mm.plan_prefill(16 * 5 + 3, chunk_tokens=32)
    assert plan.kind == "pipelined" and plan.l1_pages == 2 and plan.l2_prefetch == 4 and sum(plan.chunk_schedule) == 83
    mm.migrate(a[0], Tier.L2_CPU)
    assert mm.free_pages() == 3 and mm.used[Tier.L2_CPU] == 1
    with pytest.raises(MemoryError):
        mm.allocate(4)
    mm.finalize_session("s", a[1:3], 30)
    assert mm.claim_session("s", 7) == (a[1:3], 30) and mm.claim_session("s", 8) == ([], 0)
    mm.finalize_session("s", a[1:4], 45)
    assert mm.claim_session("s", 9)[1] == 45
    w = mm.allocate(1, pipeline=KvPipeline.WORKING)
    mm.record_entropy(a[4], 6.0); mm.record_entropy(a[5], 1.0); mm.record_entropy(w[0], 0.1)
    assert mm.entropy_victims(2) == [w[0], a[4]]
    mm.drop_session("s")
    assert a[1] not in mm.table


def test_codecs_crc_and_swap_file(tmp_path):
    data = bytes([0] * 500 + [7] * 300 + list(range(200)))
    assert rle_bitpack_decode(rle_bitpack_encode(data)) == data and len(rle_bitpack_encode(data)) < len(data)
    for c in CompressionCodec:
        if c != CompressionCodec.NVCOMP_ANS:
            assert decompress(compress(data, c), c) == data
    assert crc16_ccitt(b"123456789") == 0x29B1
    f = NvmeSwapFile(str(tmp_path / "swap.bin"), slot_bytes=1024, slots=4)
    s = f.write(data, CompressionCodec.ZSTD)
    assert f.read(s, release=False) == data
    raw = bytearray(os.pread(f.fd, 16, s * f.slot_bytes)); raw[12] ^= 0xFF
    os.pwrite(f.fd, bytes(raw), s * f.slot_bytes)
    with pytest.raises(Exception):
        f.read(s)
    f.close()


def test_three_tier_swap_round_trip_and_policy(tmp_path):
    pool = torch.arange(6 * 2 * 16 * 8, dtype=torch.float32).reshape(6, 2, 16, 8).to(torch.bfloat16)
    orig = pool.clone()
    sw = ThreeTierSwap(pool, host_slots=3, swap_path=str(tmp_path / "kv.swap"), nvme_slots=2)
    for k in range(6):
        sw.register(k, k, importance=50 if k < 2 else 200)
    for _ in range(60):
        sw.tick()
    cmds = sw.eviction_pass(hbm_used_ratio=0.95)
    assert sorted(k for _, k in cmds) == [0, 1] and sw.records[0].tier == StorageTier.DRAM
    assert sw.eviction_pass(hbm_used_ratio=0.5) == []
    pool[0].zero_(); pool[1].zero_()
    sw.execute(DmaCommand.EVICT_TO_NVME, 0)
    assert sw.records[0].tier == StorageTier.NVME
    sw.execute(DmaCommand.PROMOTE_TO_HBM, 0)                     # NVMe -> DRAM -> HBM
    sw.execute(DmaCommand.PROMOTE_TO_HBM, 1)
    r0, r1 = sw.records[0], sw.records[1]
    assert r0.tier == r1.tier == StorageTier.HBM
    torch.testing.assert_close(pool[r0.location], orig[0]); torch.testing.assert_close(pool[r1.location], orig[1])
    assert sw.stats == {"evict_dram": 2, "evict_nvme": 1, "promote_hbm": 2, "promote_dram": 1}
    assert ThreeTierSwap.swap_in_urgency(0.5, 0.2, StorageTier.HBM) > ThreeTierSwap.swap_in_urgency(0.5, 0.2, StorageTier.NVME)
    sw.close()
    w = BackgroundWorker(lambda x: x * 2, "t"); w.start(); w.submit(21)
    assert w.done.get(timeout=2)[:2] == (21, 42)
    w.submit("boom"); w.fn = lambda x: 1 / 0; assert isinstance(w.done.get(timeout=2)[2], ZeroDivisionError)
    w.stop()


def test_weight_paging_faults_retries_prefetch_and_defrag():
    loads, fail = [], {"n": 0}

    def loader(page, off):
        if fail["n"] > 0:
            fail["n"] -= 1
            raise IOError("injected")
        loads.append((page.key, off))

    t = WeightPageTable(arena_bytes=100, loader=loader, max_retries=3)
    for i in range(5):
        t.add(f"e{i}", 30)
    t.add("pinned", 10, pinned=True)
    assert t.ensure_resident("pinned") == 0 and t.ensure_resident("e0") == 10 and t.ensure_resident("e1") == 40
    t.ensure_resident("e2")
    assert t.pages["e0"].tier == Tier.L1_GPU
    t.ensure_resident("e3")                                     # evicts LRU (e0)
    assert t.pages["e0"].tier == Tier.L2_CPU and t.stats["evictions"] == 1
    fail["n"] = 2
    t.ensure_resident("e0")                                     # two failures then success
    assert t.stats["retries"] == 2 and t.pages["e0"].tier == Tier.L1_GPU
    fail["n"] = 5
    with pytest.raises(PageFaultError):
        t.ensure_resident("e4")
    fail["n"] = 0
    plan = t.plan_step(7, ["e4", "e0"])
    assert plan.to_load == ["e4"] and plan.stall_bytes == 30 and plan.to_evict == []   # the failed load left room
    t.enqueue_prefetch("e4", 0.9); t.enqueue_prefetch("e1", 0.1)
    assert t.run_prefetch(budget_bytes=30) == ["e4"]
    missing = [k for k, p in t.pages.items() if p.tier != Tier.L1_GPU][0]
    plan = t.plan_step(8, [missing])
    assert plan.to_load == [missing] and len(plan.to_evict) == 1 and "pinned" not in plan.to_evict
    t.evict(sorted(t.resident(), key=lambda p: p.offset)[1].key)
    moved = t.defragment()
    offs = sorted(p.offset for p in t.resident())
    assert moved >= 1 and offs[0] == 0 and t.fragmentation() == 0.0
    big = WeightPageTable(arena_bytes=10, loader=loader)
    big.add("x", 50)
    with pytest.raises(PageFaultError):
        big.ensure_resident("x")


def test_kv_optimizer_scores_and_tiers():
    assert importance_score(0.0, 0.9, 255, 1.0) == 230 and importance_score(6.93, 0.1, 0, 0.0) == 0
    assert is_sink_page(100, True) and is_sink_page(201, False) and not is_sink_page(200, False)
    assert [decide_tier(s) for s in (250, 160, 100, 50, 20, 5)] == [PrecisionTier.FP16, PrecisionTier.FP8, PrecisionTier.KIVI4,
                                                                    PrecisionTier.KIVI2, PrecisionTier.SPARSE, PrecisionTier.EVICTED]
    assert decide_tier(5, KvPipeline.CONVERSATION) == PrecisionTier.FP8
    assert decide_tier(50, KvPipeline.WORKING, layer=0, num_layers=30) == PrecisionTier.FP8
    assert decide_tier(50, KvPipeline.WORKING, layer=29, num_layers=30) == PrecisionTier.KIVI2
    k, v = torch.randn(16, 64), torch.randn(16, 64)
    sizes = []
    for t in (PrecisionTier.FP16, PrecisionTier.FP8, PrecisionTier.KIVI4, PrecisionTier.KIVI2, PrecisionTier.SPARSE, PrecisionTier.EVICTED):
        kk, vv, n = requantize_page(k, v, t)
        sizes.append(n)
        assert kk.shape == k.shape
    assert sizes == sorted(sizes, reverse=True) and sizes[-1] == 0


def test_observer_request_state_and_chunking():
    ob = BasicObserver()
    ob.record_attention(4.0, 0.5, alpha=1.0)
    st = ob.system_state(free_pages=10, total_pages=100, fragmentation=0.2, running=3, waiting=1)
    assert abs(st.memory_pressure - 0.9) < 1e-6 and st.logits_entropy == 4.0 and st.running == 3
    rs = RequestStateTable(4)
    rs.assign(1, request_id=77, max_tokens=2, eos_token=9)
    assert rs.advance(1, 5) == 0 and rs.rec[1]["phase"] == Phase.DECODE
    assert rs.advance(1, 9) == int(ExitFlag.EOS | ExitFlag.LENGTH) and rs.rec[1]["phase"] == Phase.FINISHED
    rs.open_port(1, 3); assert rs.rec[1]["bus_ports"] == 8
    rs.release(1); assert rs.rec[1]["request_id"] == 0
    cc = ChunkedConfig()
    assert (cc.adaptive_chunk(0.1), cc.adaptive_chunk(0.9), cc.adaptive_chunk(0.5)) == (64, 2048, 1056)
    sch = ChunkedPrefillScheduler()
    b = sch.compose(list(range(3000)), [(1, 5000), (2, 100)], memory_pressure_ratio=0.5, slots_in_use=10, slots_total=20)
    assert b.budget == 2048 and len(b.decode_ids) == 1228 and b.prefill == [(1, 512), (2, 100)] and b.compact_required
    assert compaction_plan([0, 3, 5]) == [(3, 1), (5, 2)]
    sk = SwiftKvPlan(32)
    assert sk.cut_layer == 16 and len(sk.skipped_layers()) == 16 and sk.prefill_flop_ratio() == 0.5


def test_mtp_controller_follows_the_reference_policy():
    """alpha 0.1 from 0.5; three low steps in a row switch the heads off; five plain steps switch them back on; the depth
    follows the average (> 0.8 full, > 0.5 two, > 0.3 one)."""
    from gllm_b200.speculative.mtp_executor import MtpController
    c = MtpController(4)
    assert c.enabled and c.draft_len() == 1 and abs(c.ema - 0.5) < 1e-9            # 0.5 is not > 0.5
    c.update(4, 4)
    assert abs(c.ema - 0.55) < 1e-6 and c.draft_len() == 2
    for _ in range(30):
        c.update(4, 4)
    assert c.ema > 0.8 and c.draft_len() == 4
    assert c.update(0, 4) and c.update(1, 4) and not c.update(0, 4)               # the third low step in a row
    assert c.draft_len() == 0
    for _ in range(4):
        assert not c.update(0, 0)
    assert c.update(0, 0) and c.enabled                                            # the fifth plain step
    c2 = MtpController(4)
    c2.update(0, 4); c2.update(4, 4); c2.update(0, 4); c2.update(0, 4)
    assert c2.enabled                                                              # the streak was broken
