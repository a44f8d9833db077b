import torch

from gllm_b200.engine.arbiter import (Archetype, HardwareSummary, InferenceMode, OverlapHint, ScenarioHint, StrategyArbiter,
                                      archetype_of)
from gllm_b200.engine.batch_context import BatchContext
from gllm_b200.engine.callbacks import (CallbackAction, CallbackChain, CallbackTable, EarlyExitCallback, GateSkipCallback,
                                        MidLayerEncodeCallback, ProbeVetoCallback, RagInjectCallback, port_layers,
                                        SLOT_GUARDRAIL)
from gllm_b200.engine.guard import CanaryDeviceBuffer, GuardedHostBuffer, NanTrap
from gllm_b200.engine.weight_blob import WeightBlob
from gllm_b200.models.config import preset
import pytest


def test_arbiter_plans():
    arb = StrategyArbiter(HardwareSummary(gpus=8))
    q8 = preset("qwen3-8b")
    assert archetype_of(q8) == Archetype.DENSE_MEDIUM and archetype_of(preset("qwen3-30b-a3b")) == Archetype.MOE
    assert archetype_of(preset("deepseek-v3")) == Archetype.MLA_MOE and archetype_of(preset("tiny-bert")) == Archetype.ENCODER
    thr = arb.arbitrate(q8, InferenceMode.THROUGHPUT)
    lat = arb.arbitrate(q8, InferenceMode.LATENCY)
    assert thr.tp == 1 and lat.tp >= 2 and lat.max_num_seqs < thr.max_num_seqs and lat.speculative and not thr.speculative
    big = arb.arbitrate(preset("llama-3-70b"), InferenceMode.THROUGHPUT)
    assert big.tp >= 2 and big.fused_collectives
    moe = arb.arbitrate(preset("qwen3-30b-a3b"))
    assert moe.ep == 8 and moe.tp == 1
    ds = arb.arbitrate(preset("deepseek-v3"))
    assert ds.ep == 8 and ds.weight_dtype == "fp8"
    iso = arb.arbitrate(preset("llama-3-70b"), overlap=OverlapHint.PREFER_ISOLATED)
    assert not iso.fused_collectives
    lc = arb.arbitrate(q8, scenario=ScenarioHint.LONG_CONTEXT)
    assert lc.kv_dtype == "fp8"
    one = StrategyArbiter(HardwareSummary(gpus=1)).arbitrate(q8)
    assert (one.tp, one.pp, one.ep) == (1, 1, 1) and not one.fused_collectives


def test_callback_chain_and_table():
    assert port_layers(32) == {"rag_inject": 16, "early_exit": 25, "intent": 24, "guardrail": 30, "sg_detect": 16}
    h = torch.randn(4, 8)
    enc = MidLayerEncodeCallback(2)
    rag = RagInjectCallback(2, torch.ones(8), scale=2.0)
    chain = CallbackChain([enc, rag])
    assert chain.layers_of_interest(6) == [2]
    r = chain.run("pre", 2, h)
    assert r.action == CallbackAction.REPLACE and torch.allclose(r.hidden[-1], h[-1] + 2) and torch.equal(r.hidden[0], h[0])
    chain.run("post", 2, h); assert torch.equal(enc.captured, h)
    ee = EarlyExitCallback(layer=5)
    assert ee.post_layer(4, h).action == CallbackAction.CONTINUE
    assert ee.post_layer(5, h * 1.001).action == CallbackAction.EXIT_EARLY
    assert ee.post_layer(4, h).action == CallbackAction.CONTINUE and ee.post_layer(5, -h).action == CallbackAction.CONTINUE
    veto = ProbeVetoCallback(1, weight=torch.ones(8) * 10, threshold=0.5)
    chain2 = CallbackChain([MidLayerEncodeCallback(1), veto])
    assert chain2.callbacks[0] is veto                                     # priority order
    assert chain2.run("post", 1, torch.ones(2, 8)).action == CallbackAction.VETO
    assert chain2.run("post", 1, -torch.ones(2, 8)).action == CallbackAction.CONTINUE
    gs = GateSkipCallback([3]); gs.pre_layer(3, h)
    assert torch.equal(gs.post_layer(3, h * 5).hidden, h)
    t = CallbackTable(); t.register(SLOT_GUARDRAIL, lambda x: x + 1)
    assert t.call(SLOT_GUARDRAIL, 1) == 2 and t.call(0) is None
    with pytest.raises(IndexError):
        t.register(8, print)


def test_batch_context_layout():
    bc = BatchContext(8)
    seqs = [dict(request_id=7, q_len=1, ctx_len=100, slot=0, temperature=0.7, top_k=0, top_p=1.0, eos=2, generated=5, max_tokens=256),
            dict(request_id=9, q_len=33, ctx_len=33, slot=1, temperature=0.0, top_k=40, top_p=0.9, eos=2, generated=0, max_tokens=16)]
    bc.fill(seqs, step=12, seed=99, max_blocks=64)
    assert bc.nbytes() == 96 + 128 and int(bc.header["num_tokens"][0]) == 34 and int(bc.header["num_decode"][0]) == 1
    assert int(bc.seqs[1]["q_start"]) == 1 and int(bc.seqs[1]["block_table_off"]) == 64
    raw = bytes(bc.buf[:96].numpy())
    assert raw[:4] == (0x474C4C4D).to_bytes(4, "little")
    sp = bc.sampling_params()
    assert sp.shape == (2, 4) and sp[1].tolist() == [0.0, 40.0, 0.8999999761581421, 2.0]
    assert bc.upload("cpu").numel() == bc.nbytes()


def test_guards_nan_trap_and_blob(tmp_path):
    g = GuardedHostBuffer(5000)
    t = g.tensor()
    t.fill_(7)
    assert t.numel() == 5000 and int(t.sum()) == 35000
    lo, hi = g.guard_addresses()
    assert g.address - lo == 4096 and hi > g.address + 5000 - 1
    c = CanaryDeviceBuffer(100, torch.float32, "cpu")
    c.data.fill_(1.0); assert c.intact()
    c.raw[c.pad + 400] = 0; assert not c.intact()
    trap = NanTrap(enabled=True, dump_dir=str(tmp_path))
    trap.check("ok", torch.ones(3))
    with pytest.raises(FloatingPointError):
        trap.check("bad", torch.tensor([1.0, float("nan")]))
    assert (tmp_path / "bad.pt").exists()
    NanTrap(enabled=False).check("bad", torch.tensor([float("inf")]))
    ts = {f"L{l}.{n}": torch.randn(3, 5).to(dt) for l in range(2) for n, dt in (("w", torch.bfloat16), ("s", torch.float32))}
    ts["lm_head"] = torch.randn(7)
    blob = WeightBlob.pack(ts)
    for n, t0 in ts.items():
        assert torch.equal(blob.view(n), t0) and blob.entries[n].offset % 256 == 0
    assert blob.layer_stride("L0.", "L1.") == 512 and blob.layer_stride("L0.", "lm") is None
    assert blob.offset_table()[0][0] == "L0.w" and blob.total_bytes() % 256 == 0


def test_coordinators_and_backend_context():
    from gllm_b200.backend import BackendContext
    from gllm_b200.engine.coordinators import Coordinators
    from gllm_b200.engine.executor import EngineConfig
    from gllm_b200.models.decoder import DecoderModel
    from gllm_b200.models.weights import RandomWeights
    from gllm_b200.parallel.config import PdRole
    cfg = preset("tiny-llama")
    model = DecoderModel(cfg, RandomWeights(cfg, "cpu", torch.float32, seed=1), device="cpu", dtype=torch.float32, max_positions=128)
    ctx = BackendContext("cpu")
    assert ctx.backend.info.name == "cpu" and 0.0 <= ctx.backend.get_memory_pressure() <= 1.0
    eng = ctx.build_executor(model, EngineConfig(max_num_seqs=2, max_model_len=128, max_batch_tokens=64, num_pages=32))
    co = Coordinators.of(eng, pd_role=PdRole.COLLOCATED)
    rid = co.dispatch.enqueue([1, 2, 3, 4], max_tokens=3, temperature=0.0, eos_ids=[])
    assert co.dispatch.queue_depths() == {"waiting": 1, "running": 0} and co.dispatch.phases()["prefill"]
    st = co.observability.capture()
    assert st.waiting == 1 and co.kv.occupancy() == 0.0 and co.compute.tp_mode() == "none"
    co.inference.drain()
    assert len(eng.results[rid].token_ids) == 3 and co.model_ctx.config is cfg
    assert co.kv.plan()["store_heads"] == list(range(cfg.num_kv_heads))
    # three-tier accounting over the engine's pools, and the prefill page plan it gives
    from gllm_b200.scheduler.types import Tier
    mem = co.kv.memory
    assert mem.cap[Tier.L1_GPU] == 32 and mem.used[Tier.L1_GPU] == 32 - eng.batcher.num_free_pages
    assert co.kv.plan_prefill(100).kind == "fully_resident"
    big = co.kv.plan_prefill(16 * 40)
    assert big.kind == "pipelined" and big.l2_prefetch > 0 and sum(big.chunk_schedule) == 16 * 40
    swp = _tiny_engine(num_pages=22, swap_space_pages=12)
    m2 = swp.coordinators.kv.memory
    assert m2.cap[Tier.L2_CPU] == 12 and m2.used[Tier.L2_CPU] == 0


def test_engine_step_raises_on_a_device_status_code_and_fails_the_requests():
    """The serving path consults the kernels' status word every step: a non-zero code (injected on the host here) fails
    the running requests instead of committing the step's tokens, and the engine says why."""
    from gllm_b200.engine.executor import EngineConfig, LLMEngine
    from gllm_b200.models.decoder import DecoderModel
    from gllm_b200.models.weights import RandomWeights
    from gllm_b200.ops._native import DeviceStatusError
    cfg = preset("tiny-qwen3")
    model = DecoderModel(cfg, RandomWeights(cfg, "cpu", torch.float32, seed=0), device="cpu", dtype=torch.float32,
                         max_positions=128)
    eng = LLMEngine(model, EngineConfig(max_num_seqs=4, max_model_len=64, max_batch_tokens=64, prefill_chunk=64))
    a = eng.add_request([5, 6, 7, 8], max_tokens=4, temperature=0.0, eos_ids=[])
    b = eng.add_request([9, 10, 11], max_tokens=4, temperature=0.0, eos_ids=[])
    eng.step()                                     # prefill
    eng.step()                                     # one clean decode step
    eng.h_status[0] = 5                            # what a timed-out wait for a peer rank leaves behind
    real = eng._run_decode

    def run_decode_keeping_status(plan):           # the download of a real step would overwrite the injected word
        out = real(plan)
        eng.h_status[0] = 5
        return out
    eng._run_decode = run_decode_keeping_status
    with pytest.raises(DeviceStatusError, match="peer rank"):
        eng.step()
    assert eng.unhealthy and "5" in eng.unhealthy
    assert not eng.reqs                            # nothing keeps running on a rank in this state
    ra, rb = eng.results[a], eng.results[b]
    assert ra.finish_reason.startswith("error: rank unhealthy") and rb.finish_reason.startswith("error")
    assert len(ra.token_ids) <= 2                  # the faulty step's tokens were not committed


def _tiny_engine(**kw):
    from gllm_b200.engine.executor import EngineConfig, LLMEngine
    from gllm_b200.models.decoder import DecoderModel
    from gllm_b200.models.weights import RandomWeights
    cfg = preset("tiny-qwen3")
    model = DecoderModel(cfg, RandomWeights(cfg, "cpu", torch.float32, seed=0), device="cpu", dtype=torch.float32,
                         max_positions=256)
    base = dict(max_num_seqs=6, max_model_len=160, max_batch_tokens=256, prefill_chunk=128, enable_prefix_cache=False)
    base.update(kw)
    return LLMEngine(model, EngineConfig(**base))


def test_swap_tier_under_memory_pressure_gives_the_unconstrained_tokens(tmp_path):
    """A KV pool smaller than the working set: sequences chosen by the eviction policy leave for pinned host memory
    (and, beyond its size, for the NVMe file) and come back later; the tokens equal those of a run with enough pages."""
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, 1000, (n,), generator=g).tolist() for n in (40, 33, 48, 37, 45, 30)]
    want = [r.token_ids for r in _tiny_engine(num_pages=128).generate_batch(prompts, max_tokens=40, temperature=0.0, eos_ids=[])]
    eng = _tiny_engine(num_pages=22, swap_space_pages=12, swap_path=str(tmp_path / "kv.swap"), swap_nvme_pages=64)
    got = [r.token_ids for r in eng.generate_batch(prompts, max_tokens=40, temperature=0.0, eos_ids=[])]
    assert got == want
    assert eng.stats["swap_outs"] > 0 and eng.stats["swap_ins"] == eng.stats["swap_outs"]
    assert eng.kv_swap.stats["pages_out"] == eng.kv_swap.stats["pages_in"] > 0
    assert eng.kv_swap.stats["to_nvme"] > 0              # host space (12 pages) overflowed into the file tier
    assert not eng.kv_swap.keys and not eng.kv_swap.swap.records
    # the same pool without a swap tier falls back to recompute-style preemption, also with the right tokens
    rec = _tiny_engine(num_pages=22)
    assert [r.token_ids for r in rec.generate_batch(prompts, max_tokens=40, temperature=0.0, eos_ids=[])] == want
    assert rec.stats["preemptions"] > 0 and rec.stats.get("swap_outs", 0) == 0


def test_speculative_decoding_in_the_engine_equals_plain_greedy():
    """Prompt-lookup drafts verified by one forward per step: the same tokens as plain greedy decoding, in fewer steps
    whenever drafts are accepted; acceptance statistics are kept."""
    g = torch.Generator().manual_seed(5)
    base = torch.randint(0, 1000, (12,), generator=g).tolist()
    prompts = [base * 3, torch.randint(0, 1000, (25,), generator=g).tolist(), (base[:5] * 6)[:29]]
    plain = _tiny_engine(num_pages=128)
    want = [r.token_ids for r in plain.generate_batch(prompts, max_tokens=48, temperature=0.0, eos_ids=[])]
    spec = _tiny_engine(num_pages=128, speculative_tokens=4)
    got = [r.token_ids for r in spec.generate_batch(prompts, max_tokens=48, temperature=0.0, eos_ids=[])]
    assert got == want
    st = spec.spec_stats
    assert st["steps"] > 0 and st["drafted"] > 0 and 0 <= st["accepted"] <= st["drafted"]
    assert st["emitted"] >= st["steps"]
    if st["accepted"]:
        assert spec.stats["decode_steps"] < plain.stats["decode_steps"]
    # sampling requests never speculate (the verify rule here is the greedy one)
    hot = _tiny_engine(num_pages=128, speculative_tokens=4)
    hot.generate_batch(prompts[:1], max_tokens=8, temperature=0.8, eos_ids=[])
    assert hot.spec_stats["steps"] == 0


def test_mtp_heads_in_the_model_feed_the_verify_step():
    """``mtp_proj.{d}`` heads in the checkpoint: the model emits candidates next to its main token, the next step
    verifies them in one forward, the acceptance controller adapts the depth; tokens equal plain greedy decoding."""
    from gllm_b200.engine.executor import EngineConfig, LLMEngine
    from gllm_b200.models.decoder import DecoderModel
    from gllm_b200.models.weights import RandomWeights
    cfg = preset("tiny-qwen3")
    base = RandomWeights(cfg, "cpu", torch.float32, seed=0)

    class WithMtp:           # two heads that are copies of the output head: right whenever the output repeats itself
        def has(self, n):
            return n in ("mtp_proj.0", "mtp_proj.1") or base.has(n)

        def get(self, n):
            if n.startswith("mtp_proj."):
                return base.get("lm_head") if base.has("lm_head") else base.get("embed_tokens")
            return base.get(n)
    model = DecoderModel(cfg, WithMtp(), device="cpu", dtype=torch.float32, max_positions=256)
    assert len(model.mtp_heads) == 2
    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(0, 1000, (n,), generator=g).tolist() for n in (36, 25, 29)]
    ec = dict(max_num_seqs=6, max_model_len=160, max_batch_tokens=256, prefill_chunk=128, num_pages=128)
    want = [r.token_ids for r in LLMEngine(model, EngineConfig(**ec)).generate_batch(prompts, max_tokens=48, temperature=0.0, eos_ids=[])]
    eng = LLMEngine(model, EngineConfig(mtp_depth=2, **ec))
    assert eng.mtp is not None and eng.mtp.depth == 2
    got = [r.token_ids for r in eng.generate_batch(prompts, max_tokens=48, temperature=0.0, eos_ids=[])]
    assert got == want
    assert eng.spec_stats["drafted"] > 0 and 0.0 <= eng.mtp.controller.ema <= 1.0
    # the single-request entry point with the reference's result fields
    r = LLMEngine(model, EngineConfig(mtp_depth=2, **ec)).generate_with_mtp(prompts[0], max_tokens=48, eos_ids=[])
    assert r["committed_tokens"] == want[0] and r["total_mtp_candidates"] > 0
    assert 0 <= r["total_mtp_accepted"] <= r["total_mtp_candidates"] and r["steps"] > 0
    r0 = LLMEngine(model, EngineConfig(**ec)).generate_with_mtp(prompts[0], max_tokens=48, eos_ids=[])
    assert r0["committed_tokens"] == want[0] and r0["total_mtp_candidates"] == 0


def test_prefill_and_decode_roles_hand_requests_over_with_their_kv_pages():
    """A prefill_only engine and a decode_only engine joined by a link produce what one collocated engine produces;
    the decode side computes only the partial last page of each prompt."""
    from gllm_b200.engine.pd import InProcessPdLink
    g = torch.Generator().manual_seed(9)
    prompts = [torch.randint(0, 1000, (n,), generator=g).tolist() for n in (50, 33, 64, 19)]
    want = [r.token_ids for r in _tiny_engine(num_pages=128).generate_batch(prompts, max_tokens=12, temperature=0.0, eos_ids=[])]
    link = InProcessPdLink()
    pre = _tiny_engine(num_pages=128, pd_role="prefill_only", enable_prefix_cache=True)
    dec = _tiny_engine(num_pages=128, pd_role="decode_only", enable_prefix_cache=True)
    pre.pd_link, dec.pd_link = link, link
    ids = [pre.add_request(p, max_tokens=12, temperature=0.0, eos_ids=[]) for p in prompts]
    first = {}
    while pre.has_work():
        for r in pre.step():
            assert r.finish_reason == "handoff" and len(r.token_ids) == 1
            first[r.request_id] = r.token_ids[0]
    assert pre.stats["decode_steps"] == 0 and pre.stats["pd_exported"] == 4
    done = {}
    for _ in range(200):
        for r in dec.step():
            done[r.request_id] = r
        if len(done) == 4:
            break
    assert [done[i].token_ids for i in ids] == want
    assert all(first[i] == want[j][0] for j, i in enumerate(ids))      # the prefill side's first token is the same one
    assert dec.stats["pd_imported"] == 4
    # 50 -> 3 cached pages (48), 33 -> 32, 64 -> 48 (one token is always left to compute), 19 -> 16
    assert [done[i].telemetry.cached_prefix_tokens for i in ids] == [48, 32, 48, 16]
    assert dec.stats["prefill_tokens"] == sum(len(p) for p in prompts) - (48 + 32 + 48 + 16)


def test_engine_buckets_follow_the_observed_batch_sizes_and_the_director():
    from gllm_b200.runtime.director import ConsensusEvent
    eng = _tiny_engine(num_pages=128, max_num_seqs=6, adaptive_buckets=True)
    assert eng._bucket(3) == 4 and eng._bucket(6) == 6 and eng.buckets.buckets[-1] == 6
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, 1000, (12,), generator=g).tolist() for _ in range(3)]
    eng.generate_batch(prompts, max_tokens=40, temperature=0.0, eos_ids=[])
    assert eng.buckets.hist.total >= 39 and eng.director_state.batch_sizes.mean() > 0
    eng._on_director_event(ConsensusEvent("bucket_drift", 0, 0.9))
    assert eng._evolve_pending
    before, after = eng.evolve_buckets()
    assert after[-1] == 6 and 3 in after or 4 in after       # three running sequences: a bucket near 3, capacity kept
    assert not eng._evolve_pending


def test_decoder_weights_live_in_one_blob():
    """With ``weight_blob=True`` the packed dense tensors of a decoder are views into one contiguous allocation with an
    offset table and a constant per-layer stride, and the model computes the same logits as without it."""
    import torch
    from gllm_b200.engine.batch import ForwardBatch
    from gllm_b200.models.config import preset
    from gllm_b200.models.decoder import DecoderModel
    from gllm_b200.models.weights import RandomWeights
    cfg = preset("tiny-qwen3")
    src = RandomWeights(cfg, "cpu", torch.float32, seed=1, std=0.05)
    a = DecoderModel(cfg, src, device="cpu", dtype=torch.float32, weight_blob=False, max_positions=64)
    b = DecoderModel(cfg, src, device="cpu", dtype=torch.float32, weight_blob=True, max_positions=64)
    assert a.blob is None and b.blob is not None
    base = b.blob.data.data_ptr()
    for lw in b.layers:
        assert base <= lw.wqkv.data_ptr() < base + b.blob.total_bytes()
        assert (lw.wqkv.data_ptr() - base) % 256 == 0
    assert b.blob.layer_stride("L0.", "L1.") > 0          # homogeneous layers: one byte distance for every tensor
    T = 9
    i32 = dict(dtype=torch.int32)
    fb = lambda: ForwardBatch(token_ids=torch.arange(T, **i32) + 3, positions=torch.arange(T, **i32),
                              slot_mapping=torch.arange(T, **i32), block_tables=torch.arange(2, **i32)[None],
                              ctx_lens=torch.tensor([T], **i32), q_start=torch.tensor([0], **i32),
                              q_len=torch.tensor([T], **i32), max_q_len=T)
    la = a.forward(fb(), a.alloc_kv_cache(2))
    lb = b.forward(fb(), b.alloc_kv_cache(2))
    torch.testing.assert_close(la, lb)


def test_engine_keeps_the_per_slot_request_table():
    """LLMEngine mirrors every running request in the 32-byte-per-slot record table (phase, counters, exit flags): the
    record appears with the first prefill chunk, advances with every token and is released when the request ends."""
    import torch
    from gllm_b200.engine.executor import EngineConfig, LLMEngine
    from gllm_b200.models.config import preset
    from gllm_b200.models.decoder import DecoderModel
    from gllm_b200.models.weights import RandomWeights
    from gllm_b200.scheduler.request_state import Phase
    cfg = preset("tiny-qwen3")
    model = DecoderModel(cfg, RandomWeights(cfg, "cpu", torch.float32, seed=2, std=0.05), device="cpu",
                         dtype=torch.float32, max_positions=128)
    eng = LLMEngine(model, EngineConfig(max_num_seqs=4, max_model_len=64, max_batch_tokens=64, num_pages=32))
    a = eng.add_request([3, 4, 5, 6], max_tokens=5, temperature=0.0, eos_ids=[])
    b = eng.add_request([7, 8, 9], max_tokens=2, temperature=0.0, eos_ids=[])
    eng.step()          # prefill: both get a slot and their first token
    rec = eng.request_states()
    live = {int(r["request_id"]): r for r in rec if r["phase"] != Phase.IDLE}
    assert set(live) == {a, b}
    assert live[a]["generated"] == 1 and live[a]["max_tokens"] == 5 and live[a]["phase"] == Phase.DECODE
    eng.step()
    rec = eng.request_states()
    assert [int(r["generated"]) for r in rec if int(r["request_id"]) == a and r["phase"] != Phase.IDLE] == [2]
    done = eng.run_until_done()
    assert {r.request_id for r in done} == {a, b}
    assert all(r["phase"] == Phase.IDLE for r in eng.request_states())


def test_kv_distribution_modes_move_cached_prefixes_between_engines():
    """MIRROR: a finished conversation's pages are copied into the peers' prefix caches; ON_DEMAND: a rank that misses a
    prefix fetches it from the peer that has it; LOCAL: nothing moves. The next turn on the other engine starts from
    the cached pages and gives the tokens of an engine that computed everything itself."""
    from gllm_b200.parallel.config import KvDistMode
    from gllm_b200.parallel.pd import KvDistributor
    g = torch.Generator().manual_seed(11)
    turn1 = torch.randint(0, 1000, (53,), generator=g).tolist()
    for mode in (KvDistMode.MIRROR, KvDistMode.ON_DEMAND, KvDistMode.LOCAL):
        a, b = _tiny_engine(num_pages=64, enable_prefix_cache=True), _tiny_engine(num_pages=64, enable_prefix_cache=True)
        dist_ = KvDistributor({0: a, 1: b}, mode)
        r1 = a.generate_batch([turn1], max_tokens=12, temperature=0.0, eos_ids=[])[0]
        convo = turn1 + r1.token_ids
        moved = dist_.after_finish(0, convo)
        turn2 = convo + torch.randint(0, 1000, (9,), generator=g).tolist()
        fetched = dist_.before_admit(1, turn2)
        r2 = b.generate_batch([turn2], max_tokens=6, temperature=0.0, eos_ids=[])[0]
        want = _tiny_engine(num_pages=64).generate_batch([turn2], max_tokens=6, temperature=0.0, eos_ids=[])[0]
        assert r2.token_ids == want.token_ids
        full = len(convo) // 16 * 16
        if mode == KvDistMode.MIRROR:
            assert moved == full // 16 and fetched == 0 and r2.telemetry.cached_prefix_tokens == full
        elif mode == KvDistMode.ON_DEMAND:
            assert moved == 0 and fetched == full // 16 and r2.telemetry.cached_prefix_tokens == full
            assert dist_.stats["fetches"] == 1
        else:
            assert moved == 0 and fetched == 0 and r2.telemetry.cached_prefix_tokens == 0


def test_eagle_head_drafts_are_verified_by_the_target():
    """An EAGLE head attached to the engine: drafts continue the target's last hidden feature; whatever the head
    proposes (here an untrained one, and one that is made to agree with the target), the tokens equal plain greedy
    decoding, and agreeing drafts shorten the run."""
    from gllm_b200.speculative.heads import EagleHead
    g = torch.Generator().manual_seed(6)
    prompts = [torch.randint(0, 1000, (n,), generator=g).tolist() for n in (19, 33)]
    plain = _tiny_engine(num_pages=64)
    want = [r.token_ids for r in plain.generate_batch(prompts, max_tokens=12, temperature=0.0, eos_ids=[])]
    eng = _tiny_engine(num_pages=64)
    m = eng.model
    head = EagleHead(m.cfg.hidden_size, m.embed, m.lm_head, m.final_norm, seed=1, dtype=torch.float32)
    eng.attach_eagle(head, depth=3)
    got = [r.token_ids for r in eng.generate_batch(prompts, max_tokens=12, temperature=0.0, eos_ids=[])]
    assert got == want
    st = eng.spec_stats
    assert st["steps"] > 0 and st["drafted"] > 0 and not eng._eagle_feat       # features dropped with the requests

    class Oracle:      # a "head" that knows the target's continuation: every draft is accepted
        def __init__(self, answers):
            self.answers = answers

        def draft(self, feature, token, depth):
            t = int(token[0])
            for seq in self.answers:
                if t in seq:
                    i = seq.index(t)
                    return [torch.tensor([x]) for x in seq[i + 1:i + 1 + depth]]
            return []
    eng2 = _tiny_engine(num_pages=64)
    eng2.attach_eagle(Oracle(want), depth=3)
    got2 = [r.token_ids for r in eng2.generate_batch(prompts, max_tokens=12, temperature=0.0, eos_ids=[])]
    assert got2 == want
    if all(len(set(w)) == len(w) for w in want):      # unambiguous look-ups: every proposed token was right
        assert eng2.spec_stats["accepted"] == eng2.spec_stats["drafted"] > 0
        assert eng2.stats["decode_steps"] < plain.stats["decode_steps"]


def test_abort_cancels_waiting_and_running_requests():
    eng = _tiny_engine(num_pages=64, max_num_seqs=2)
    g = torch.Generator().manual_seed(1)
    rids = [eng.add_request(torch.randint(0, 1000, (20,), generator=g).tolist(), max_tokens=30, temperature=0.0, eos_ids=[])
            for _ in range(3)]                       # two run, one waits
    for _ in range(4):
        eng.step()
    assert eng.abort(rids[0], "cancelled by the caller") and eng.abort(rids[2]) and not eng.abort(12345)
    eng.run_until_done()
    a, b, c = (eng.results[r] for r in rids)
    assert a.finish_reason == "cancelled by the caller" and 0 < len(a.token_ids) < 30
    assert c.finish_reason == "aborted" and len(c.token_ids) == 0
    assert b.finish_reason == "length" and len(b.token_ids) == 30
    assert eng.batcher.num_free_pages == eng.batcher.num_total_pages or eng.cfg.enable_prefix_cache


def test_replica_router_keeps_conversations_on_their_replica_and_fetches_pages_when_it_cannot():
    from gllm_b200.engine.serving import ReplicaRouter, ServingLoop
    g = torch.Generator().manual_seed(21)
    a, b = _tiny_engine(num_pages=96, enable_prefix_cache=True), _tiny_engine(num_pages=96, enable_prefix_cache=True)
    router = ReplicaRouter([ServingLoop(a), ServingLoop(b)])
    turn1 = torch.randint(0, 1000, (50,), generator=g).tolist()
    other = torch.randint(0, 1000, (45,), generator=g).tolist()
    f1 = router.submit(turn1, max_tokens=10, temperature=0.0, eos_ids=[])
    f2 = router.submit(other, max_tokens=10, temperature=0.0, eos_ids=[])          # the less loaded replica takes it
    r1, r2 = f1.result(timeout=120), f2.result(timeout=120)
    assert {f1.replica, f2.replica} == {0, 1}
    convo = turn1 + r1.token_ids
    turn2 = convo + torch.randint(0, 1000, (7,), generator=g).tolist()
    f3 = router.submit(turn2, max_tokens=5, temperature=0.0, eos_ids=[])
    r3 = f3.result(timeout=120)
    assert f3.replica == f1.replica and router.stats["affinity_hits"] >= 1          # the turn follows its conversation
    assert r3.telemetry.cached_prefix_tokens == len(convo) // 16 * 16
    want = _tiny_engine(num_pages=96).generate_batch([turn2], max_tokens=5, temperature=0.0, eos_ids=[])[0]
    assert r3.token_ids == want.token_ids
    # the owner is "saturated": the other replica gets the request and fetches the conversation's pages first
    router.max_in_flight = 0
    turn3 = turn2 + r3.token_ids + [5, 6, 7]
    f4 = router.submit(turn3, max_tokens=4, temperature=0.0, eos_ids=[])
    r4 = f4.result(timeout=120)
    assert router.stats["fetched_pages"] > 0 and r4.telemetry.cached_prefix_tokens > 0
    want4 = _tiny_engine(num_pages=96).generate_batch([turn3], max_tokens=4, temperature=0.0, eos_ids=[])[0]
    assert r4.token_ids == want4.token_ids
    router.shutdown()


def test_speculation_switches_off_when_drafts_keep_failing_and_for_large_batches():
    g = torch.Generator().manual_seed(8)
    prompt = torch.randint(0, 1000, (24,), generator=g).tolist()
    want = _tiny_engine(num_pages=64).generate_batch([prompt], max_tokens=40, temperature=0.0, eos_ids=[])[0].token_ids

    class Wrong:                      # a draft source that is always wrong
        def extend(self, toks):
            pass

        def lookup(self, k, top=1):
            return [[1001 % 1000 + 7] * k]
    eng = _tiny_engine(num_pages=64, speculative_tokens=4)
    rid = eng.add_request(prompt, max_tokens=40, temperature=0.0, eos_ids=[])
    eng._spec_idx[rid] = Wrong()
    eng.run_until_done()
    assert eng.results[rid].token_ids == want
    st = eng.spec_stats
    assert eng.spec_state.controller.draft_len() == 0            # the acceptance average fell below the switch-off level
    assert 0 < st["steps"] < 30 and st["accepted"] <= 2          # it stopped drafting long before the request ended
    # more decoding sequences than speculative_max_batch: the plain (captured) decode step runs instead
    many = _tiny_engine(num_pages=256, speculative_tokens=4, speculative_max_batch=32, max_num_seqs=40)
    base = torch.randint(0, 1000, (6,), generator=g).tolist()
    outs = many.generate_batch([base * 3 + [i] for i in range(36)], max_tokens=6, temperature=0.0, eos_ids=[])
    assert all(len(r.token_ids) == 6 for r in outs)
    assert many.spec_stats["steps"] < many.stats["decode_steps"]


def test_adaptive_prefill_chunk_follows_free_pages():
    """Plenty of free pages: the prompt is prefilled in one chunk of up to ``prefill_chunk`` tokens; with the pool
    partly taken the chunk shrinks (between the minimum of 64 and the maximum, by the share of free pages: two prefill
    steps here), and the tokens do not change."""
    g = torch.Generator().manual_seed(13)
    long_prompt = torch.randint(0, 1000, (100,), generator=g).tolist()
    filler = [torch.randint(0, 1000, (60,), generator=g).tolist() for _ in range(7)]
    base = dict(max_num_seqs=8, max_model_len=200, max_batch_tokens=512, prefill_chunk=128, enable_prefix_cache=False)
    want = _tiny_engine(num_pages=256, **base).generate_batch([long_prompt], max_tokens=4, temperature=0.0, eos_ids=[])[0]
    roomy = _tiny_engine(num_pages=256, adaptive_prefill_chunk=True, **base)
    r = roomy.generate_batch([long_prompt], max_tokens=4, temperature=0.0, eos_ids=[])[0]
    assert r.token_ids == want.token_ids and roomy.stats["prefill_steps"] == 1
    tight = _tiny_engine(num_pages=48, adaptive_prefill_chunk=True, **base)
    for p in filler:
        tight.add_request(p, max_tokens=40, temperature=0.0, eos_ids=[])
    tight.step()                             # the fillers' prompts hold 28 of the 48 pages now
    assert 0.25 < tight.batcher.num_free_pages / tight.batcher.num_total_pages < 0.5      # chunk cap about 80 tokens
    before = tight.stats["prefill_steps"]
    rid = tight.add_request(long_prompt, max_tokens=4, temperature=0.0, eos_ids=[])
    while rid not in tight.results:
        tight.step()
    assert tight.results[rid].token_ids == want.token_ids
    assert tight.stats["prefill_steps"] - before >= 2                                    # 80 + 20 tokens
