import math

import torch

from gllm_b200.models import gemma_ops as G
from gllm_b200.models.config import preset


def test_norms_and_dual_rope():
    x = torch.randn(5, 4, 64) * 3
    q = G.qk_norm_weightless(x)
    torch.testing.assert_close(q.pow(2).mean(-1), torch.ones(5, 4), rtol=1e-3, atol=1e-3)
    torch.testing.assert_close(G.value_norm(x).pow(2).mean(-1), torch.ones(5, 4), rtol=1e-3, atol=1e-3)
    assert [l for l in range(10) if G.layer_uses_global_rope(l)] == [4, 9]
    assert G.dual_rope_theta(3, 1e6, 1e4) == 1e4 and G.dual_rope_theta(4, 1e6, 1e4) == 1e6
    cfg = preset("tiny-llama")
    cfg.rope_local_theta = 100.0
    cg, sg, cl, sl = G.build_dual_rope_tables(cfg, 32)
    assert cg.shape == cl.shape and not torch.allclose(cg[5], cl[5])


def test_laurel_altup_and_ple():
    torch.manual_seed(0)
    T, H, n = 6, 16, 4
    x, a = torch.randn(T, H), torch.randn(T, H)
    lw = G.LaurelWeights(torch.zeros(4, H), torch.zeros(H, 4), torch.ones(H))
    torch.testing.assert_close(G.laurel(x, a, lw), (x + a) / math.sqrt(2))          # zero low-rank branch
    lw = G.LaurelWeights(torch.randn(4, H), torch.randn(H, 4), torch.ones(H))
    assert not torch.allclose(G.laurel(x, a, lw), (x + a) / math.sqrt(2))
    w = G.AltUpWeights(router=torch.randn(n, H), predict=torch.zeros(n * n, n), correct=torch.zeros(n, n),
                       router_norm=torch.ones(H), out_scale=torch.ones(H))
    streams = torch.randn(n, T, H)
    pred = G.altup_predict(streams, w)
    torch.testing.assert_close(pred, streams)                                         # zero predictor = identity
    act = streams[0] + 1.0
    cor = G.altup_correct(pred, act, w)
    torch.testing.assert_close(cor[0], act)                                           # active stream takes the layer output
    torch.testing.assert_close(cor[2], streams[2] + 1.0)                              # innovation spread with coefficient 1
    w.predict = torch.randn(n * n, n) * 0.1
    assert not torch.allclose(G.altup_predict(streams, w), streams)
    table = torch.arange(10 * 3 * 4, dtype=torch.float32).reshape(10, 12)
    e = G.ple_gather(table, torch.tensor([2, 7]), layer=1, num_layers=3)
    torch.testing.assert_close(e, table[[2, 7], 4:8] * 2.0)
    inj = G.altup_inject(cor, e.new_ones(T, H), w)
    torch.testing.assert_close(inj[0], cor[0]); torch.testing.assert_close(inj[1], cor[1] + 1.0)


def test_logit_softcap_in_the_gemm_op_cpu():
    """ops.gemm(softcap=c) == c * tanh(x / c) on the CPU oracle path (the CUDA path does it in the GEMM epilogue)."""
    import torch
    from gllm_b200 import ops
    torch.manual_seed(0)
    a = torch.randn(5, 64).to(torch.bfloat16)
    w = torch.randn(32, 64).to(torch.bfloat16)
    got = ops.gemm(a, w, out_dtype=torch.float32, softcap=7.0)
    x = a.float() @ w.float().t()
    torch.testing.assert_close(got, torch.tanh(x / 7.0) * 7.0)


def _tiny_shared_kv_model(fused, seed=0, perturb=False):
    import torch
    from gllm_b200.models.config import ModelConfig
    from gllm_b200.models.decoder import DecoderModel
    from gllm_b200.models.weights import RandomWeights
    cfg = ModelConfig(arch="llama", hidden_size=256, num_layers=4, num_heads=2, num_kv_heads=1, head_dim=128,
                      intermediate_size=512, vocab_size=300, max_position_embeddings=128, rms_norm_eps=1e-6,
                      num_kv_shared_layers=2)
    src = RandomWeights(cfg, "cpu", torch.bfloat16, seed=seed, std=0.05)
    if perturb:           # other keys / values for the shared layers: they must not matter
        base_get = src.get

        def get(name):
            t = base_get(name)
            if name.startswith(("L2.", "L3.")) and name.rsplit(".", 1)[-1] in ("k_proj", "v_proj"):
                return t + 1.0
            return t
        src.get = get
    return cfg, DecoderModel(cfg, src, device="cpu", dtype=torch.bfloat16, fused=fused, max_positions=128)


def _run_tokens(model, ids, kv=None, start=0):
    import torch
    from gllm_b200.engine.batch import ForwardBatch
    n = len(ids)
    total = start + n
    kv = kv or model.alloc_kv_cache(8)
    i32 = dict(dtype=torch.int32)
    fb = ForwardBatch(token_ids=torch.tensor(ids, **i32), positions=torch.arange(start, total, **i32),
                      slot_mapping=torch.arange(start, total, **i32), block_tables=torch.arange(8, **i32)[None],
                      ctx_lens=torch.tensor([total], **i32), q_start=torch.tensor([0], **i32),
                      q_len=torch.tensor([n], **i32), max_q_len=n, logits_rows=torch.tensor([n - 1]))
    return model.forward(fb, kv).float()[0, :300], kv


def test_shared_kv_donor_layers():
    """The last two layers of a four-layer model project no keys / values and attend over layer 1's cache: the donor
    map, the aliasing of the caches, independence from the shared layers' own K / V weights, fused and unfused paths
    agreeing, and prefill + one more token matching a single longer prefill."""
    import torch
    cfg, m = _tiny_shared_kv_model(fused=True)
    assert [cfg.kv_donor(i) for i in range(4)] == [None, None, 1, 1]
    assert m.layers[2].n_kv == 0 and m.layers[2].wqkv.shape[0] == 2 * 128
    kv = m.alloc_kv_cache(8)
    assert kv[2] is kv[1] and kv[3] is kv[1] and kv[0] is not kv[1]
    ids = [5, 17, 250, 3, 99, 42, 7]
    ref, _ = _run_tokens(m, ids)
    _, m2 = _tiny_shared_kv_model(fused=True, perturb=True)
    got, _ = _run_tokens(m2, ids)
    torch.testing.assert_close(got, ref)
    _, mu = _tiny_shared_kv_model(fused=False)
    got_u, _ = _run_tokens(mu, ids)
    assert torch.nn.functional.cosine_similarity(got_u, ref, dim=0) > 0.995
    _, kv = _run_tokens(m, ids[:-1])
    step, _ = _run_tokens(m, ids[-1:], kv=kv, start=len(ids) - 1)
    assert torch.nn.functional.cosine_similarity(step, ref, dim=0) > 0.999


def _g3n_cfg(**kw):
    from gllm_b200.models.config import preset
    cfg = preset("tiny-qwen3")
    cfg.num_layers = 3
    for k, v in kw.items():
        setattr(cfg, k, v)
    return cfg


def _g3n_batch(ids, start, n, pages=4, decode=False):
    from gllm_b200.engine.batch import ForwardBatch
    i32 = lambda v: torch.tensor(v, dtype=torch.int32)
    pos = list(range(start, start + n))
    return ForwardBatch(token_ids=ids[start:start + n], positions=i32(pos), slot_mapping=i32(pos),
                        block_tables=torch.arange(pages, dtype=torch.int32)[None], ctx_lens=i32([start + n]),
                        q_start=i32([0]), q_len=i32([n]), max_q_len=n, is_decode=decode)


def test_altup_with_neutral_weights_is_the_plain_decoder():
    """The stream bookkeeping inside the decoder: with a silent AltUp router (prediction = identity, correction = the
    layer's innovation on every stream), identity projections and unit output scale all streams follow the active one,
    so the logits equal the plain model's."""
    from gllm_b200.models.decoder import DecoderModel
    from gllm_b200.models.weights import RandomWeights

    class Neutral(RandomWeights):
        def get(self, name):
            base = name.rsplit(".", 1)[-1]
            if base == "altup_router":
                return torch.zeros(self.shape_of(name))
            if base == "altup_out_scale":
                return torch.ones(self.shape_of(name))
            if name.startswith("altup_proj.") or name.startswith("altup_unproj."):
                return torch.eye(self.cfg.hidden_size)
            return super().get(name)

    plain_cfg, alt_cfg = _g3n_cfg(), _g3n_cfg(altup_num_inputs=3)
    plain = DecoderModel(plain_cfg, RandomWeights(plain_cfg, "cpu", torch.float32, seed=2, std=0.05), device="cpu",
                         dtype=torch.float32, max_positions=64)
    alt = DecoderModel(alt_cfg, Neutral(alt_cfg, "cpu", torch.float32, seed=2, std=0.05), device="cpu", dtype=torch.float32,
                       max_positions=64)
    assert not alt.fused and len(alt.altup_proj) == 2
    ids = (torch.arange(20, dtype=torch.int32) * 7 + 1) % plain_cfg.vocab_size
    want = plain.forward(_g3n_batch(ids, 0, 20), plain.alloc_kv_cache(4))
    got = alt.forward(_g3n_batch(ids, 0, 20), alt.alloc_kv_cache(4))
    torch.testing.assert_close(got, want, rtol=1e-4, atol=1e-5)


def test_gemma3n_structure_prefill_and_decode_agree():
    """AltUp (4 streams), LAuReL and per-layer embeddings with random weights: the logits of position t are the same
    whether the prompt is prefilled at once, in two chunks, or the last token is decoded on the cached pages; every
    feature changes the logits; the model serves through the engine."""
    from gllm_b200.models.decoder import DecoderModel
    from gllm_b200.models.weights import RandomWeights
    feats = dict(altup_num_inputs=4, laurel_rank=8, ple_dim=16)
    cfg = _g3n_cfg(**feats)
    src = RandomWeights(cfg, "cpu", torch.float32, seed=5, std=0.05)
    m = DecoderModel(cfg, src, device="cpu", dtype=torch.float32, max_positions=64)
    ids = (torch.arange(24, dtype=torch.int32) * 5 + 3) % cfg.vocab_size
    full = m.forward(_g3n_batch(ids, 0, 24), m.alloc_kv_cache(4))
    assert torch.isfinite(full).all()
    kv = m.alloc_kv_cache(4)
    a = m.forward(_g3n_batch(ids, 0, 17), kv)
    b = m.forward(_g3n_batch(ids, 17, 6), kv)
    c = m.forward(_g3n_batch(ids, 23, 1, decode=True), kv)
    torch.testing.assert_close(torch.cat([a, b, c]), full, rtol=2e-4, atol=2e-4)
    base = DecoderModel(_g3n_cfg(), RandomWeights(_g3n_cfg(), "cpu", torch.float32, seed=5, std=0.05), device="cpu",
                        dtype=torch.float32, max_positions=64).forward(_g3n_batch(ids, 0, 24), m.alloc_kv_cache(4))
    for name, val in feats.items():
        one = _g3n_cfg(**{name: val})
        lg = DecoderModel(one, RandomWeights(one, "cpu", torch.float32, seed=5, std=0.05), device="cpu", dtype=torch.float32,
                          max_positions=64).forward(_g3n_batch(ids, 0, 24), m.alloc_kv_cache(4))
        if name == "ple_dim":       # per-layer embeddings enter through the non-active streams only: silent without AltUp
            torch.testing.assert_close(lg, base)
        else:
            assert not torch.allclose(lg, base), name
    from gllm_b200.engine.executor import EngineConfig, LLMEngine
    eng = LLMEngine(m, EngineConfig(max_num_seqs=2, max_model_len=64, max_batch_tokens=32, prefill_chunk=32, num_pages=16))
    out = eng.generate_batch([ids[:9].tolist(), ids[:20].tolist()], max_tokens=4, temperature=0.0, eos_ids=[])
    assert [len(r.token_ids) for r in out] == [4, 4]


def test_dual_rope_rotates_sliding_layers_with_the_local_base():
    """Gemma-3 style: layers with a sliding window rotate q / k with ``rope_local_theta``, global layers with
    ``rope_theta``. Checked against the same model where the pattern makes every layer global / every layer local."""
    from gllm_b200.models.decoder import DecoderModel
    from gllm_b200.models.weights import RandomWeights
    ids = (torch.arange(30, dtype=torch.int32) * 3 + 2) % 1000

    def logits(**kw):
        cfg = _g3n_cfg(num_layers=2, **kw)
        m = DecoderModel(cfg, RandomWeights(cfg, "cpu", torch.float32, seed=7, std=0.05), device="cpu", dtype=torch.float32,
                         max_positions=64)
        return m, m.forward(_g3n_batch(ids, 0, 30), m.alloc_kv_cache(4))

    # window 64 >= sequence: the window itself changes nothing, only the rotation base can
    m, mixed = logits(rope_theta=1e6, rope_local_theta=1e4, sliding_window=64, attention_pattern=[1, 0])
    assert m.cos_local is not None and m._rope(0)[0] is m.cos_local and m._rope(1)[0] is m.cos
    _, all_global = logits(rope_theta=1e6, rope_local_theta=1e4, sliding_window=64, attention_pattern=[0, 0])
    _, plain_global = logits(rope_theta=1e6)
    torch.testing.assert_close(all_global, plain_global)
    _, all_local = logits(rope_theta=1e6, rope_local_theta=1e4, sliding_window=64, attention_pattern=[1, 1])
    _, plain_local = logits(rope_theta=1e4)
    torch.testing.assert_close(all_local, plain_local)
    assert not torch.allclose(mixed, all_global) and not torch.allclose(mixed, all_local)
    # layer 0 local + layer 1 global equals a hand-built pair of tables used per layer
    import gllm_b200.models.rope as rope
    cfg = m.cfg
    lo = rope.build_tables(cfg, 64, "cpu", theta=1e4)
    torch.testing.assert_close(m.cos_local, lo[0])
