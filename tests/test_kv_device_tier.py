"""The 4-bit KV tier on the device: packed page layout, unpacking, attention over mixed block tables, and the
serving engine packing preempted sequences instead of copying them to the host."""
import pytest
import torch

from gllm_b200.kv_cache import device_tier as DT
from gllm_b200.kv_cache.quant import kivi_dequantize, kivi_quantize_page
from gllm_b200.models.config import preset


def _cache(pages, n_kv, D, dtype, seed=0):
    g = torch.Generator().manual_seed(seed)
    c = torch.randn(pages, 2, n_kv, 16, D, generator=g)
    c[:, 0, :, :, 3] *= 8.0          # an outlier key channel: its own range keeps the others fine-grained
    return c.to(dtype)


def test_packed_layout_size_and_error_bound():
    n_kv, D = 2, 128
    cache = _cache(6, n_kv, D, torch.float32)
    pool = torch.zeros(4, DT.page_bytes(n_kv, D), dtype=torch.uint8)
    assert DT.page_bytes(n_kv, D) == n_kv * 2624 and DT.page_bytes(n_kv, D) * 3 < cache[0].numel() * 2
    DT.pack_pages(cache, pool, [1, 4], [3, 0])
    out = torch.zeros_like(cache)
    DT.unpack_pages(out, pool, [3, 0], [2, 5])
    for src, dst in ((1, 2), (4, 5)):
        k, v = cache[src, 0], cache[src, 1]
        k_step = (k.amax(1) - k.amin(1)) / 15            # per channel  [n_kv, D]
        v_step = (v.amax(2) - v.amin(2)) / 15            # per token    [n_kv, 16]
        assert ((out[dst, 0] - k).abs() <= 0.51 * k_step[:, None, :] + 2e-3).all()
        assert ((out[dst, 1] - v).abs() <= 0.51 * v_step[..., None] + 2e-3).all()
    assert out[[0, 1, 3, 4]].abs().sum() == 0                # only the named pages were written
    # the same grid as the host-side KIVI statement (up to the fp16 rounding of scale and zero)
    ref = kivi_quantize_page(cache[1, 0, 0], cache[1, 1, 0], bits=4)
    rk, rv = kivi_dequantize(ref)
    for mine, theirs in ((out[2, 0, 0], rk), (out[2, 1, 0], rv)):
        d = (mine - theirs).abs()
        assert d.mean() < 0.01 and (d > 0.05).float().mean() < 0.01      # a few codes flip at rounding ties


def test_constant_groups_survive_exactly():
    cache = torch.full((1, 2, 1, 16, 64), 0.75)
    pool = torch.zeros(1, DT.page_bytes(1, 64), dtype=torch.uint8)
    DT.pack_pages(cache, pool, [0], [0])
    out = torch.zeros_like(cache)
    DT.unpack_pages(out, pool, [0], [0])
    assert torch.equal(out, cache)


def test_tiered_attention_reads_packed_pages_in_place():
    n_q, n_kv, D = 4, 2, 64
    cache = _cache(10, n_kv, D, torch.float32, seed=1) * 0.5
    pool = torch.zeros(6, DT.page_bytes(n_kv, D), dtype=torch.uint8)
    DT.pack_pages(cache, pool, [2, 7, 8], [4, 1, 0])
    # sequence 0: pages 2 (packed), 3 (bf16), 7 (packed); sequence 1: page 8 (packed), 5 (bf16)
    bt = torch.tensor([[-5, 3, -2], [-1, 5, 0]], dtype=torch.int32)
    q_len = torch.tensor([5, 1], dtype=torch.int32)
    ctx = torch.tensor([44, 20], dtype=torch.int32)
    q_start = torch.tensor([0, 5], dtype=torch.int32)
    q = torch.randn(6, n_q * D, generator=torch.Generator().manual_seed(2))
    got = DT.paged_attention_tiered(q, cache, pool, bt, q_start, q_len, ctx, max_q_len=5, n_q=n_q, n_kv=n_kv, scale=0.125)
    # oracle: the same attention over a cache whose packed pages were unpacked in place
    deq = cache.clone()
    DT.unpack_pages(deq, pool, [4, 1, 0], [2, 7, 8])
    from gllm_b200.ops.attention import attention_ref
    want = attention_ref(q, deq, torch.tensor([[2, 3, 7], [8, 5, 0]], dtype=torch.int32), q_start, q_len, ctx, n_q, n_kv,
                         0.125, True, 0, None)
    torch.testing.assert_close(got, want, rtol=1e-5, atol=1e-5)
    exact = attention_ref(q, cache, torch.tensor([[2, 3, 7], [8, 5, 0]], dtype=torch.int32), q_start, q_len, ctx, n_q, n_kv,
                          0.125, True, 0, None)
    assert (got - exact).abs().max() < 0.15 and not torch.equal(got, exact)      # 4-bit pages: close, not equal


def test_engine_packs_preempted_sequences_on_the_device():
    """Memory pressure with a device pool: victims are packed to 4 bits on the device (no host copy) and resume from
    the unpacked pages; when the pool is full the host tier takes the rest. Every request still completes with the
    requested number of tokens, and most tokens equal the unconstrained run (the tier is lossy)."""
    from tests.test_engine_extras import _tiny_engine
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, 1000, (n,), generator=g).tolist() for n in (40, 33, 48, 37, 45, 30)]
    want = [r.token_ids for r in _tiny_engine(num_pages=128).generate_batch(prompts, max_tokens=40, temperature=0.0, eos_ids=[])]
    eng = _tiny_engine(num_pages=22, swap_space_pages=64, kv_kivi_pool_pages=8)
    res = eng.generate_batch(prompts, max_tokens=40, temperature=0.0, eos_ids=[])
    assert [len(r.token_ids) for r in res] == [40] * 6
    st = eng.kv_swap.stats
    assert st["packed_seqs"] > 0 and st["packed_pages"] == st["unpacked_pages"] > 0
    assert st["pages_out"] > 0                               # the 8-slot pool overflowed into the host tier
    assert not eng.kv_swap.packed and len(eng.kv_swap.device_tier.free) == 8
    assert eng.kv_swap.sink_pages == 1 and not eng.kv_swap.sink_keys and not eng.kv_swap.swap.records   # sink pages came back too
    same = sum(a == b for r, w in zip(res, want) for a, b in zip(r.token_ids, w))
    assert same >= 0.5 * 240, same


def test_sessions_and_important_requests_keep_full_precision():
    """The KV optimiser decides where a victim waits: a session's pages (conversation pipeline: never below fp8) and
    requests marked important go to the host unchanged; the rest may be packed to 4 bits on the device."""
    from gllm_b200.kv_cache.header import PrecisionTier
    from tests.test_engine_extras import _tiny_engine
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, 1000, (n,), generator=g).tolist() for n in (40, 33, 48, 37, 45, 30)]
    want = [r.token_ids for r in _tiny_engine(num_pages=128).generate_batch(prompts, max_tokens=40, temperature=0.0, eos_ids=[])]
    eng = _tiny_engine(num_pages=22, swap_space_pages=64, kv_kivi_pool_pages=32)
    rids = [eng.add_request(p, max_tokens=40, temperature=0.0, eos_ids=[], session_id=f"chat-{i}") for i, p in enumerate(prompts)]
    assert eng._swap_tier(rids[0]) <= PrecisionTier.FP8
    while eng.has_work():
        eng.step()
    got = [eng.results[r].token_ids for r in rids]
    assert got == want                                     # nothing was quantised: same tokens as without pressure
    assert eng.kv_swap.stats["packed_seqs"] == 0 and eng.kv_swap.stats["pages_out"] > 0
    # without a session the same request may wait in 4 bits, unless its importance says otherwise
    rid = eng.add_request(prompts[0], max_tokens=4, temperature=0.0, eos_ids=[])
    assert eng._swap_tier(rid) == PrecisionTier.KIVI4
    eng.kv_importance[rid] = 230
    assert eng._swap_tier(rid) == PrecisionTier.FP16
    while eng.has_work():
        eng.step()
    assert rid not in eng.kv_importance and not eng._sessions


@pytest.mark.gpu
def test_device_kernels_match_the_cpu_statement():
    from gllm_b200.ops import _native as nv
    dev = torch.device("cuda")
    for n_kv, D in ((2, 128), (3, 64)):
        cache = _cache(12, n_kv, D, torch.bfloat16, seed=4)
        pool_cpu = torch.zeros(8, DT.page_bytes(n_kv, D), dtype=torch.uint8)
        DT.pack_pages(cache, pool_cpu, [1, 4, 9, 11], [3, 0, 7, 2])
        cache_d = cache.to(dev)
        pool_d = torch.zeros(8, DT.page_bytes(n_kv, D), dtype=torch.uint8, device=dev)
        DT.pack_pages(cache_d, pool_d, [1, 4, 9, 11], [3, 0, 7, 2])
        torch.cuda.synchronize()
        diff = (pool_d.cpu() != pool_cpu).float().mean().item()
        assert diff < 0.002, f"packed bytes differ in {diff:.4%} of the pool"     # ties of the rounding at most
        out_d = torch.zeros_like(cache_d)
        DT.unpack_pages(out_d, pool_d, [3, 0, 7, 2], [0, 5, 6, 10])
        out_c = torch.zeros_like(cache)
        DT.unpack_pages(out_c, pool_d.cpu(), [3, 0, 7, 2], [0, 5, 6, 10])
        torch.testing.assert_close(out_d.float().cpu(), out_c.float(), rtol=1e-2, atol=1e-2)
        # attention over mixed block tables
        n_q = 2 * n_kv
        bt = torch.tensor([[-4, 6, -8, 5], [10, -1, 0, 0]], dtype=torch.int32)
        q_len = torch.tensor([7, 1], dtype=torch.int32)
        ctx = torch.tensor([60, 29], dtype=torch.int32)
        q_start = torch.tensor([0, 7], dtype=torch.int32)
        q = (torch.randn(8, n_q * D, generator=torch.Generator().manual_seed(5)) * 0.5).to(torch.bfloat16)
        want = DT.paged_attention_tiered(q.float(), out_c.float() + cache.float() * 0, pool_d.cpu(), bt, q_start, q_len, ctx,
                                         max_q_len=7, n_q=n_q, n_kv=n_kv, scale=D ** -0.5)
        got = DT.paged_attention_tiered(q.to(dev), out_d, pool_d, bt.to(dev), q_start.to(dev), q_len.to(dev), ctx.to(dev),
                                        max_q_len=7, n_q=n_q, n_kv=n_kv, scale=D ** -0.5)
        torch.testing.assert_close(got.float().cpu(), want, rtol=2e-2, atol=2e-2)
    assert nv.device_error() == 0


def test_kv_page_telemetry_feeds_headers_and_importance():
    """After a decode step the sampled pass recomputes the last layer's attention of every running sequence from the
    workspace queries and the cache pages: its output equals what the step itself computed (so the rows, positions and
    pages line up), the per-page masses sum to one, the 64-byte headers carry the telemetry, and every request gets an
    importance score the swap tier decision reads."""
    from tests.test_engine_extras import _tiny_engine
    from gllm_b200.kv_cache.header import PrecisionTier
    eng = _tiny_engine(num_pages=64, kv_telemetry_every=1)
    g = torch.Generator().manual_seed(2)
    rids = [eng.add_request(torch.randint(0, 1000, (n,), generator=g).tolist(), max_tokens=6, temperature=0.0, eos_ids=[])
            for n in (37, 18)]
    checked = 0
    while eng.has_work():
        before = eng.kv_telemetry.samples
        eng.step()
        if eng.kv_telemetry.samples > before:
            lo = eng.kv_telemetry.last_out
            mine = lo["out"].reshape(-1)
            theirs = eng.model._ws.attn[lo["slot"]].float()[:mine.numel()]
            if eng.model._ws.attn.shape[0] and torch.isfinite(theirs).all():
                torch.testing.assert_close(mine, theirs, rtol=1e-4, atol=1e-5)
                checked += 1
    assert checked > 0 and eng.kv_telemetry.samples >= 4
    h = eng.kv_telemetry.headers.h
    used = h[h["ref_count"] > 0]
    assert len(used) >= 3 and set(int(x) for x in used["sequence_id"]) <= set(rids)
    assert (used["importance"] > 0).any() and all(0 <= int(t) <= int(PrecisionTier.EVICTED) for t in used["precision_tier"])
    assert (used["centroid"].astype("float32") >= 0).all() and float(used["entropy"].astype("float32").max()) <= 6.94
    # masses of one sequence's pages sum to one (checked through the stats function directly)
    from gllm_b200.engine.kv_telemetry import attention_page_stats
    kv = eng.kv_caches[-1]
    q = torch.randn(eng.model.n_q_local * kv.shape[-1])
    st = attention_page_stats(q, kv, [3, 1, 2], 40, eng.model.n_q_local, eng.model.n_kv_local, 0.1)
    assert abs(float(st["mass"].sum()) - 1.0) < 1e-5 and st["entropy"].shape == (3,) and float(st["softmax_max"].max()) <= 1.0


def test_per_page_tiers_split_a_victim_between_the_pool_and_the_host():
    """With page telemetry the KV optimiser's tier of every page decides where it waits: pages it wants above 4 bits
    (and the sink page) go to the host unchanged, the others are packed; they come back in logical order."""
    from gllm_b200.kv_cache.header import PrecisionTier
    from tests.test_engine_extras import _tiny_engine
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, 1000, (n,), generator=g).tolist() for n in (40, 33, 48, 37, 45, 30)]
    want = [r.token_ids for r in _tiny_engine(num_pages=128).generate_batch(prompts, max_tokens=40, temperature=0.0, eos_ids=[])]
    # every page lossless (the policy says FP16 for all): the pool is never used, tokens are exact
    eng = _tiny_engine(num_pages=22, swap_space_pages=64, kv_kivi_pool_pages=32, kv_telemetry_every=1)
    assert eng.kv_swap.page_tier is not None
    eng.kv_swap.page_tier = lambda page: PrecisionTier.FP16
    got = [r.token_ids for r in eng.generate_batch(prompts, max_tokens=40, temperature=0.0, eos_ids=[])]
    assert got == want and eng.kv_swap.stats["packed_pages"] == 0 and eng.kv_swap.stats["pages_out"] > 0
    # odd pages lossless, even pages packed: both tiers are used for the same victim
    eng2 = _tiny_engine(num_pages=22, swap_space_pages=64, kv_kivi_pool_pages=32)
    eng2.kv_swap.page_tier = lambda page: PrecisionTier.FP16 if page % 2 else PrecisionTier.KIVI4
    res = eng2.generate_batch(prompts, max_tokens=40, temperature=0.0, eos_ids=[])
    st = eng2.kv_swap.stats
    assert [len(r.token_ids) for r in res] == [40] * 6
    assert st["packed_pages"] == st["unpacked_pages"] > 0 and st["pages_out"] == st["pages_in"] > 0
    assert not eng2.kv_swap.layout and not eng2.kv_swap.packed and not eng2.kv_swap.swap.records
    assert len(eng2.kv_swap.device_tier.free) == 32
