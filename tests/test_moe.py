"""MoE block on CPU: routing semantics, permutation into 128-row expert blocks, and the full layer against
the reference's dense-masked formulation (loop over all experts with gate masks)."""
import torch
import torch.nn.functional as F

from gllm_b200.models.config import preset
from gllm_b200.models.decoder import DecoderModel
from gllm_b200.models.weights import RandomWeights
from gllm_b200.ops import moe as M


def test_route_softmax_topk_renorm_and_sigmoid_bias():
    torch.manual_seed(0)
    lg = torch.randn(9, 16)
    ids, w = M.route_ref(lg, 4)
    p = torch.softmax(lg, -1)
    tv, ti = torch.topk(p, 4, -1)
    assert torch.equal(ids.long(), ti)
    torch.testing.assert_close(w, tv / tv.sum(-1, keepdim=True))
    assert torch.allclose(w.sum(-1), torch.ones(9))
    ids2, w2 = M.route_ref(lg, 4, norm_topk=False)
    torch.testing.assert_close(w2, tv)
    bias = torch.zeros(16); bias[5] = 10.0
    ids3, w3 = M.route_ref(lg, 2, scoring="sigmoid", sel_bias=bias, scale=2.5)
    assert (ids3[:, 0] == 5).all()                                   # the bias steers selection ...
    s = torch.sigmoid(lg)
    picked = torch.gather(s, 1, ids3.long())
    torch.testing.assert_close(w3, picked / picked.sum(-1, keepdim=True) * 2.5)   # ... but not the weights


def test_permute_blocks_belong_to_one_expert():
    torch.manual_seed(1)
    T, k, H, E = 37, 2, 64, 6
    x = torch.randn(T, H)
    ids = torch.randint(0, E, (T, k), dtype=torch.int32)
    ws = M.MoeWorkspace(T, k, H, 32, E, "cpu", torch.float32)
    M.permute(x, None, ids, ws, 0, E)
    offs = ws.offsets.tolist()
    assert all(o % 128 == 0 for o in offs) and offs[-1] == int(ws.total_rows[0])
    dest = ws.dest[:T * k].reshape(T, k)
    for t in range(T):
        for j in range(k):
            d, e = int(dest[t, j]), int(ids[t, j])
            assert offs[e] <= d < offs[e + 1] and torch.equal(ws.a_perm[d], x[t])
            assert int(ws.blk_group[d // 128]) == e
    assert len(set(dest.reshape(-1).tolist())) == T * k
    assert (ws.blk_group[offs[-1] // 128:] == -1).all()
    # expert-parallel view: only experts [2, 4) are local, other pairs get dest -1
    ws2 = M.MoeWorkspace(T, k, H, 32, 2, "cpu", torch.float32)
    M.permute(x, None, ids, ws2, 2, 2)
    local = (ids >= 2) & (ids < 4)
    assert torch.equal(ws2.dest[:T * k].reshape(T, k) >= 0, local)


def test_moe_layer_matches_dense_masked_reference_and_generates():
    cfg = preset("tiny-moe")
    cfg.num_shared_experts = 1
    src = RandomWeights(cfg, "cpu", torch.float32, seed=1, std=0.05)
    m = DecoderModel(cfg, src, device="cpu", dtype=torch.float32, max_positions=256)
    x = torch.randn(11, cfg.hidden_size)
    p = "L1."
    h = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + cfg.rms_norm_eps) * src.get(p + "post_attn_norm")
    probs = torch.softmax(h @ src.get(p + "router").t(), -1)
    w, ids = torch.topk(probs, cfg.num_experts_per_tok, -1)
    w = w / w.sum(-1, keepdim=True)
    ffn = lambda pre, v: (F.silu(v @ src.get(pre + "gate_proj").t()) * (v @ src.get(pre + "up_proj").t())) @ src.get(pre + "down_proj").t()
    want = x + ffn(p + "shared_expert.", h)
    for e in range(cfg.num_experts):
        want = want + ((w * (ids == e)).sum(-1, keepdim=True)) * ffn(f"{p}experts.{e}.", h)
    got = x.clone()
    m.layers[1].moe.forward_unfused(m, got, h, 11)
    torch.testing.assert_close(got, want, rtol=1e-4, atol=1e-5)
    from gllm_b200.engine.executor import EngineConfig, LLMEngine
    eng = LLMEngine(m, EngineConfig(max_num_seqs=4, max_model_len=128, max_batch_tokens=64, prefill_chunk=32))
    out = eng.generate_batch([[1, 2, 3, 4, 5], list(range(40))], max_tokens=4, temperature=0.0, eos_ids=[])
    assert [len(r.token_ids) for r in out] == [4, 4]
    # the observability coordinator sampled the routing for the load balancer while the engine ran
    obs = eng.coordinators.observability
    assert obs.eplb is not None and obs.eplb_state["totals"].sum() > 0
    assert obs.eplb_state["imbalance"] >= 1.0 and isinstance(obs.eplb_state["hot_experts"], list)
    # a skewed window: one expert takes most of the tokens -> it is named hot and the placement becomes HotCold
    from gllm_b200.parallel.config import MoePlacement
    skew = torch.ones(cfg.num_experts, dtype=torch.int64)
    skew[2] = 50 * cfg.num_experts
    obs.eplb.samples.clear()
    obs.eplb.record(skew)
    m._moe_ws[next(iter(m._moe_ws))].last_ids = torch.full((4, cfg.num_experts_per_tok), 2, dtype=torch.int32)
    st = obs.capture_expert_load()
    assert st["hot_experts"] == [2] and st["placement"] == MoePlacement.HOT_COLD and st["imbalance"] > 2.0


def test_paged_experts_match_the_resident_model():
    """Experts paged in from host memory (fewer device slots than experts: several waves per layer, evictions, the
    cross-layer prefetcher) give the logits of the model with every expert resident, in the fused-layout (block
    table over slots) and through the serving engine."""
    cfg = preset("tiny-moe")
    cfg.num_shared_experts = 1
    src = RandomWeights(cfg, "cpu", torch.float32, seed=1, std=0.05)
    full = DecoderModel(cfg, src, device="cpu", dtype=torch.float32, max_positions=256)
    paged = DecoderModel(cfg, src, device="cpu", dtype=torch.float32, max_positions=256, expert_slots=3)
    assert cfg.num_experts > 3 and paged.expert_pager is not None
    moe_layers = [lw.moe for lw in paged.layers if lw.moe is not None]
    assert all(m.w_gate_up is None and m.paged.slots == 3 for m in moe_layers)
    from gllm_b200.engine.batch import ForwardBatch

    def batch(T):
        ids = (torch.arange(T, dtype=torch.int32) * 7 + 2) % cfg.vocab_size
        return ForwardBatch(token_ids=ids, positions=torch.arange(T, dtype=torch.int32),
                            slot_mapping=torch.arange(T, dtype=torch.int32), block_tables=torch.arange(4, dtype=torch.int32)[None],
                            ctx_lens=torch.tensor([T], dtype=torch.int32), q_start=torch.tensor([0], dtype=torch.int32),
                            q_len=torch.tensor([T], dtype=torch.int32), max_q_len=T)
    for T in (23, 1, 40):
        want = full.forward(batch(T), full.alloc_kv_cache(4))
        got = paged.forward(batch(T), paged.alloc_kv_cache(4))
        torch.testing.assert_close(got, want, rtol=1e-4, atol=1e-5)
    st = paged.expert_pager.stats()
    assert st["misses"] > 0 and st["evictions"] > 0 and st["faults"] >= st["misses"]
    one = moe_layers[0].paged
    assert one.resident_bytes() * cfg.num_experts == 3 * (one.host_gu.numel() + one.host_dn.numel()) * 4
    from gllm_b200.engine.executor import EngineConfig, LLMEngine
    ecfg = dict(max_num_seqs=4, max_model_len=128, max_batch_tokens=64, prefill_chunk=32)
    prompts = [[1, 2, 3, 4, 5], list(range(40))]
    a = LLMEngine(full, EngineConfig(**ecfg)).generate_batch(prompts, max_tokens=5, temperature=0.0, eos_ids=[])
    b = LLMEngine(paged, EngineConfig(**ecfg)).generate_batch(prompts, max_tokens=5, temperature=0.0, eos_ids=[])
    assert [r.token_ids for r in a] == [r.token_ids for r in b]
    # a load that fails is retried, then reported by name
    bad = moe_layers[0].paged
    calls = {"n": 0}
    good_load = bad.handler.load_fn

    def flaky(layer, e):
        calls["n"] += 1
        if calls["n"] == 1:
            raise IOError("host copy failed")
        return good_load(layer, e)
    bad.handler.load_fn = flaky
    missing = next(e for e in range(cfg.num_experts) if e not in bad.slot_of)
    bad.ensure([missing])
    assert missing in bad.slot_of and calls["n"] == 2


def test_client_weight_paging_pages_experts():
    from gllm_b200.client import Client
    cfg = preset("tiny-moe")
    src = RandomWeights(cfg, "cpu", torch.float32, seed=1, std=0.05)
    kw = dict(device="cpu", dtype=torch.float32, max_num_seqs=2, max_model_len=128, max_batch_tokens=64)
    plain = Client.from_model(cfg, src, **kw)
    paging = Client.from_model(cfg, src, weight_paging=True, expert_slots=2, **kw)
    assert paging._state.model.expert_pager is not None and getattr(plain._state.model, "expert_pager", None) is None
    a = plain.generate("expert paging").max_tokens(5).temperature(0.0).generate().token_ids
    b = paging.generate("expert paging").max_tokens(5).temperature(0.0).generate().token_ids
    assert a == b and paging._state.model.expert_pager.stats()["misses"] > 0


def test_paged_experts_with_host_compute_for_cold_experts():
    """Hardware dispatch of a paged layer: resident experts on the device, a bounded share of the rows (experts that are
    not resident and got few rows) computed on the host from the host weights, the rest fetched. Same logits."""
    cfg = preset("tiny-moe")
    src = RandomWeights(cfg, "cpu", torch.float32, seed=1, std=0.05)
    full = DecoderModel(cfg, src, device="cpu", dtype=torch.float32, max_positions=256)
    mixed = DecoderModel(cfg, src, device="cpu", dtype=torch.float32, max_positions=256, expert_slots=2, cpu_experts=True)
    from gllm_b200.engine.batch import ForwardBatch
    T = 31
    ids = (torch.arange(T, dtype=torch.int32) * 7 + 2) % cfg.vocab_size
    mk = lambda: ForwardBatch(token_ids=ids, positions=torch.arange(T, dtype=torch.int32),
                              slot_mapping=torch.arange(T, dtype=torch.int32), block_tables=torch.arange(4, dtype=torch.int32)[None],
                              ctx_lens=torch.tensor([T], dtype=torch.int32), q_start=torch.tensor([0], dtype=torch.int32),
                              q_len=torch.tensor([T], dtype=torch.int32), max_q_len=T)
    want = full.forward(mk(), full.alloc_kv_cache(4))
    for _ in range(2):      # the second pass starts with resident experts: all three destinations are in the plan
        got = mixed.forward(mk(), mixed.alloc_kv_cache(4))
        torch.testing.assert_close(got, want, rtol=1e-4, atol=1e-5)
    pgs = [lw.moe.paged for lw in mixed.layers if lw.moe is not None]
    assert sum(pg.stats.get("host_rows", 0) for pg in pgs) > 0
    plan = pgs[0].last_plan
    assert plan.gpu_experts and plan.cpu_experts
    rows = sum(a.token_count for a in plan.gpu_experts + plan.cpu_experts + plan.remote_experts)
    assert sum(a.token_count for a in plan.cpu_experts) <= 0.2 * rows + 1e-9
    assert pgs[0].thermal.state(plan.gpu_experts[0].expert_idx) in ("hot", "warm")
