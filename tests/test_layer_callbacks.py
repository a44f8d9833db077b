"""Callback chains run inside the decoder's layer loop (eager forward) and through the serving engine."""
import torch

from gllm_b200.engine.batch import ForwardBatch
from gllm_b200.engine.callbacks import (CallbackAction, CallbackChain, EarlyExitCallback, GateSkipCallback, LayerCallback,
                                        CallbackResult, ProbeVetoCallback, RagInjectCallback)
from gllm_b200.models.config import preset
from gllm_b200.models.decoder import DecoderModel
from gllm_b200.models.weights import RandomWeights


def _batch(T, dev="cpu"):
    ids = (torch.arange(T, dtype=torch.int32) * 5 + 1) % 1000
    return ForwardBatch(token_ids=ids, positions=torch.arange(T, dtype=torch.int32),
                        slot_mapping=torch.arange(T, dtype=torch.int32), block_tables=torch.arange(4, dtype=torch.int32)[None],
                        ctx_lens=torch.tensor([T], dtype=torch.int32), q_start=torch.tensor([0], dtype=torch.int32),
                        q_len=torch.tensor([T], dtype=torch.int32), max_q_len=T)


def _model(layers=4, **kw):
    cfg = preset("tiny-qwen3")
    cfg.num_layers = layers
    src = RandomWeights(cfg, "cpu", torch.float32, seed=3, std=0.05)
    return cfg, src, DecoderModel(cfg, src, device="cpu", dtype=torch.float32, max_positions=128, **kw)


def test_injection_skip_and_early_exit_inside_the_layer_loop():
    cfg, src, m = _model()
    T = 9
    plain = m.forward(_batch(T), m.alloc_kv_cache(4)).clone()
    # an empty chain and a chain that only observes change nothing
    assert torch.equal(m.forward(_batch(T), m.alloc_kv_cache(4), callbacks=CallbackChain([])), plain)
    # RAG injection before layer 2 = the same model fed a residual stream with the vector added to its last row
    vec = torch.randn(cfg.hidden_size) * 0.5
    got = m.forward(_batch(T), m.alloc_kv_cache(4), callbacks=CallbackChain([RagInjectCallback(2, vec, 1.0)]))
    assert m.callback_action == CallbackAction.REPLACE and m.callback_info["rag_injected"]
    assert not torch.allclose(got[-1], plain[-1]) and torch.allclose(got[:-1], plain[:-1], atol=1e-5)   # causal: only the last row moves
    front = DecoderModel(cfg, src, device="cpu", dtype=torch.float32, max_positions=128, layers=range(0, 2))
    back = DecoderModel(cfg, src, device="cpu", dtype=torch.float32, max_positions=128, layers=range(2, 4))
    h = front.forward(_batch(T), front.alloc_kv_cache(4)).clone()
    h[-1] += vec
    want = back.forward(_batch(T), back.alloc_kv_cache(4), hidden_in=h)
    torch.testing.assert_close(got, want, rtol=1e-4, atol=1e-5)
    # skipping layer 1 = its output replaced by its input
    skipped = m.forward(_batch(T), m.alloc_kv_cache(4), callbacks=CallbackChain([GateSkipCallback([1])]))
    assert m.callback_info["skipped"] == 1 and not torch.allclose(skipped, plain)
    # early exit: thresholds that always hold stop the loop after the port layer; the head reads that state
    chain = CallbackChain([EarlyExitCallback(2, cos_threshold=-1.0, rho_threshold=1e9)])
    early = m.forward(_batch(T), m.alloc_kv_cache(4), callbacks=chain)
    assert m.callback_action == CallbackAction.EXIT_EARLY and m.callback_info["stopped_at"] == ("post", 2)
    three = DecoderModel(cfg, src, device="cpu", dtype=torch.float32, max_positions=128, layers=range(0, 3))
    h3 = three.forward(_batch(T), three.alloc_kv_cache(4))
    tail = DecoderModel(cfg, src, device="cpu", dtype=torch.float32, max_positions=128, layers=range(3, 4))
    # the last stage's head on the three-layer state (run its head only: no layers -> emulate by final norm + lm_head)
    from gllm_b200 import ops
    hn = ops.rmsnorm(h3, tail.final_norm, cfg.rms_norm_eps, one_plus_w=cfg.norm_one_plus_w)
    want = ops.gemm(hn, tail.lm_head, out_dtype=torch.float32, bn=256)
    torch.testing.assert_close(early, want, rtol=1e-4, atol=1e-5)


def test_replacing_rows_in_the_fused_layer_recomputes_the_norm_statistics():
    """The fused layer takes the next norm's statistics from the previous GEMM's epilogue; a callback that replaces
    the rows must not leave stale statistics behind (block-scaled model: the fused path on CPU tensors)."""
    cfg = preset("tiny-qwen3")
    cfg.hidden_size, cfg.num_heads, cfg.num_kv_heads, cfg.head_dim, cfg.intermediate_size, cfg.num_layers = 256, 2, 2, 128, 512, 3
    src = RandomWeights(cfg, "cpu", torch.float32, seed=3, std=0.05)
    m = DecoderModel(cfg, src, device="cpu", dtype=torch.float32, max_positions=128, weight_quant="mxfp8")
    assert m.fused
    plain = m.forward(_batch(7), m.alloc_kv_cache(4)).clone()

    class Same(LayerCallback):
        layers = [1]

        def pre_layer(self, layer, hidden):
            return CallbackResult(CallbackAction.REPLACE, hidden.clone())

    torch.testing.assert_close(m.forward(_batch(7), m.alloc_kv_cache(4), callbacks=CallbackChain([Same()])), plain,
                               rtol=1e-5, atol=1e-6)

    class Double(Same):
        def pre_layer(self, layer, hidden):
            return CallbackResult(CallbackAction.REPLACE, hidden * 2.0)

    doubled = m.forward(_batch(7), m.alloc_kv_cache(4), callbacks=CallbackChain([Double()]))
    assert torch.isfinite(doubled).all() and not torch.allclose(doubled, plain)


def test_semantic_gatekeeper_detect_and_inject_callback():
    from gllm_b200.sdk.semantic_gatekeeper import (KnowledgeKey, SemanticGatekeeperConfig, SemanticLevel, SgDetectInjectCallback,
                                                   SgSharedMemory)
    cfg, src, m = _model()
    T = 6
    probe = CallbackChain([])
    from gllm_b200.engine.callbacks import MidLayerEncodeCallback
    tap = MidLayerEncodeCallback(2)
    probe.add(tap)
    plain = m.forward(_batch(T), m.alloc_kv_cache(4), callbacks=probe).clone()
    here = tap.captured[-1].clone()                       # what the detect layer sees for this prompt
    mem = SgSharedMemory()
    mem.add(KnowledgeKey(0, SemanticLevel.L3_FACT, "unrelated", -here), torch.ones(cfg.hidden_size))
    mem.add(KnowledgeKey(1, SemanticLevel.L2_ENTITY, "this prompt", here), torch.full((cfg.hidden_size,), 0.3))
    sg = SgDetectInjectCallback(2, mem, SemanticGatekeeperConfig(cooldown_tokens=2))
    got = m.forward(_batch(T), m.alloc_kv_cache(4), callbacks=CallbackChain([sg]))
    assert sg.fired and sg.fired[0][0] == 1 and m.callback_info["sg_fired"] == 1 and m.callback_info["sg_similarity"] > 0.99
    assert not torch.allclose(got[-1], plain[-1])
    # cool-down: the next two forwards pass untouched
    again = m.forward(_batch(T), m.alloc_kv_cache(4), callbacks=CallbackChain([sg]))
    torch.testing.assert_close(again, plain)
    # nothing matches: no injection
    mem2 = SgSharedMemory()
    mem2.add(KnowledgeKey(0, SemanticLevel.L3_FACT, "unrelated", -here), torch.ones(cfg.hidden_size))
    quiet = SgDetectInjectCallback(2, mem2, SemanticGatekeeperConfig())
    torch.testing.assert_close(m.forward(_batch(T), m.alloc_kv_cache(4), callbacks=CallbackChain([quiet])), plain)
    assert not quiet.fired and "sg_best" in m.callback_info


def test_engine_runs_the_chain_and_a_veto_ends_the_request():
    from gllm_b200.engine.executor import EngineConfig, LLMEngine
    cfg, src, m = _model()
    base = dict(max_num_seqs=1, max_model_len=96, max_batch_tokens=64, prefill_chunk=64, enable_prefix_cache=False, num_pages=16)
    plain = LLMEngine(m, EngineConfig(**base)).generate_batch([[5, 6, 7, 8]], max_tokens=6, temperature=0.0, eos_ids=[])[0]
    vec = torch.randn(cfg.hidden_size, generator=torch.Generator().manual_seed(1)) * 4.0
    eng = LLMEngine(m, EngineConfig(callbacks=CallbackChain([RagInjectCallback(2, vec, 1.0)]), **base))
    steered = eng.generate_batch([[5, 6, 7, 8]], max_tokens=6, temperature=0.0, eos_ids=[])[0]
    assert len(steered.token_ids) == 6 and steered.token_ids != plain.token_ids      # the injection steers the tokens
    veto = CallbackChain([ProbeVetoCallback(3, torch.zeros(cfg.hidden_size), bias=10.0, threshold=0.5)])
    eng2 = LLMEngine(m, EngineConfig(callbacks=veto, **base))
    r = eng2.generate_batch([[5, 6, 7, 8]], max_tokens=6, temperature=0.0, eos_ids=[])[0]
    assert r.finish_reason == "vetoed by a layer callback" and len(r.token_ids) <= 1


def test_client_generation_with_a_chain_and_late_fusion_rag():
    from gllm_b200.client import Client
    from gllm_b200.sdk.rag import LateFusionRag
    cfg = preset("tiny-qwen3")
    cfg.num_layers = 4
    src = RandomWeights(cfg, "cpu", torch.float32, seed=3, std=0.05)
    c = Client.from_model(cfg, src, device="cpu", dtype=torch.float32, max_num_seqs=2, max_model_len=128, max_batch_tokens=64)
    plain = c.generate("what is the capital").max_tokens(6).temperature(0.0).generate()
    vec = torch.randn(cfg.hidden_size, generator=torch.Generator().manual_seed(2)) * 5.0
    steered = c.generate("what is the capital").max_tokens(6).temperature(0.0).callbacks(
        CallbackChain([RagInjectCallback(2, vec, 1.0)])).generate()
    assert steered.token_ids != plain.token_ids
    # the chain was for that call only
    assert c.generate("what is the capital").max_tokens(6).temperature(0.0).generate().token_ids == plain.token_ids
    rag = LateFusionRag(c)
    rag.index(["paris is the capital of france", "the mitochondria is the powerhouse of the cell"])
    out = rag.generate("what is the capital", top_k=1, scale=4.0, max_tokens=6, temperature=0.0)
    assert len(out.token_ids) >= 1 and c._state.engine.cfg.callbacks is None


def test_debug_serving_names_the_first_non_finite_layer():
    import pytest
    from gllm_b200.engine.executor import EngineConfig, LLMEngine
    cfg, src, m = _model()
    base = dict(max_num_seqs=1, max_model_len=96, max_batch_tokens=64, prefill_chunk=64, enable_prefix_cache=False, num_pages=16)
    eng = LLMEngine(m, EngineConfig(debug=True, **base))
    ok = eng.generate_batch([[5, 6, 7, 8]], max_tokens=3, temperature=0.0, eos_ids=[])[0]
    assert len(ok.token_ids) == 3 and eng.nan_trap.checked > 0
    # poison one weight of layer 2: the trap names that layer
    w = m.layers[2].wo
    keep = w.clone()
    w[0, 0] = float("nan")
    eng2 = LLMEngine(m, EngineConfig(debug=True, **base))
    with pytest.raises(FloatingPointError, match="hidden after layer 2"):
        eng2.generate_batch([[5, 6, 7, 8]], max_tokens=3, temperature=0.0, eos_ids=[])
    w.copy_(keep)


def test_layer_telemetry_feeds_the_epilogue_aggregator_and_its_advice_skips_a_quiet_layer():
    """The telemetry callback measures how much every layer moves the residual stream; a layer made silent (zero output
    projections) shows up as a bypass candidate, and skipping it with GateSkipCallback changes nothing."""
    from gllm_b200.engine.callbacks import LayerTelemetryCallback
    from gllm_b200.runtime.epilogue import EpilogueAggregator
    cfg, src, m = _model(layers=6)
    m.layers[3].wo.zero_()
    m.layers[3].w_down.zero_()
    agg = EpilogueAggregator(cfg.num_layers)
    plain = m.forward(_batch(9), m.alloc_kv_cache(4)).clone()
    seen = m.forward(_batch(9), m.alloc_kv_cache(4), callbacks=CallbackChain([LayerTelemetryCallback(agg)]))
    torch.testing.assert_close(seen, plain)                      # observing changes nothing
    assert set(agg.ema) == set(range(6)) and agg.ema[3].delta_rho < 1e-6 < agg.ema[2].delta_rho
    advice = agg.advice()
    assert advice.bypass_layers == [3]
    skipped = m.forward(_batch(9), m.alloc_kv_cache(4), callbacks=CallbackChain([GateSkipCallback(advice.bypass_layers)]))
    torch.testing.assert_close(skipped, plain, rtol=1e-5, atol=1e-6)
