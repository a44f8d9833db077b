import torch

from gllm_b200.client import Client
from gllm_b200.generation import HookDecision
from gllm_b200.models.config import preset
from gllm_b200.models.weights import RandomWeights
from gllm_b200.sdk import (CotConfig, CotReasoner, Guardrail, HeadRouter, IntentClassifier, IntentTracker, LateFusionRag,
                           LinearProbe, ResidualBus, Risk, SemanticGatekeeper, SemanticGatekeeperConfig, SemanticLevel, StreamGuard)
from gllm_b200.engine.callbacks import CallbackAction


def _client():
    cfg = preset("tiny-qwen3")
    return Client.from_model(cfg, RandomWeights(cfg, "cpu", torch.float32, seed=3, std=0.08), device="cpu", dtype=torch.float32,
                             max_num_seqs=4, max_model_len=512, max_batch_tokens=128)


def test_linear_probe_separates():
    torch.manual_seed(0)
    a, b = torch.randn(40, 16) + 2, torch.randn(40, 16) - 2
    p = LinearProbe.fit(torch.cat([a, b]), torch.tensor([0] * 40 + [1] * 40), ["pos", "neg"])
    assert p.predict(torch.randn(5, 16) + 2) == ["pos"] * 5 and p.predict(torch.randn(5, 16) - 2) == ["neg"] * 5
    assert abs(float(p.probabilities(a[:1]).sum()) - 1) < 1e-5


def test_cot_reasoner_budget_and_voting():
    c = _client()
    tr = CotReasoner(c, CotConfig(max_steps=2, step_tokens=4, answer_tokens=3)).reason("what is 2+2")
    assert len(tr.steps) == 2 and tr.tokens_used <= 11
    tr = CotReasoner(c, CotConfig(max_steps=5, step_tokens=4, answer_tokens=3, thinking_budget=6)).reason("q")
    assert len(tr.steps) == 2                                   # 4 + 2 tokens of budget
    calls = []
    tr = CotReasoner(c, CotConfig(max_steps=1, step_tokens=2, answer_tokens=2), verifier=lambda q, a: calls.append(a) or False).reason("q")
    assert calls and tr.steps[-1] == "[revision]"
    tr = CotReasoner(c, CotConfig(max_steps=1, step_tokens=2, answer_tokens=2, samples=3)).reason("q")
    assert sum(tr.votes.values()) == 3


def test_guardrail_intent_stream_guard():
    c = _client()
    safe = ["hello there friend", "nice weather today", "tell me a story", "good morning all"]
    unsafe = ["zzzz qqqq xxxx", "qqqq zzzz zzzz", "xxxx xxxx qqqq", "zzzz xxxx zzzz qqqq"]
    g = Guardrail.train(c, safe, unsafe)
    assert g.layer == c._st().model.cfg.num_layers - 2
    assert g.check(safe[0]).allowed and not g.check(unsafe[1]).allowed
    r, v = g.guarded_generate(unsafe[0], max_tokens=2)
    assert r is None and v.label == "unsafe"
    r, v = g.guarded_generate(safe[1], max_tokens=2, temperature=0.0)
    assert v is not None
    hook = g.hook(unsafe[0], every=1)
    assert hook.post_step(5, 1) in (HookDecision.TERMINATE, HookDecision.CONTINUE)
    # the probe inside the forward: an unsafe prompt is vetoed by its own prefill step, a safe one generates
    bad = g.guarded_generate_in_flight(unsafe[0], max_tokens=4, temperature=0.0)
    assert bad.finish_reason == "vetoed by a layer callback" and len(bad.token_ids) <= 1
    assert c._st().model.callback_info["guardrail_score"] > g.threshold
    lax = Guardrail(c, g.probe, g.layer, threshold=2.0)          # a threshold no score reaches: nothing is vetoed
    good = lax.guarded_generate_in_flight(safe[1], max_tokens=4, temperature=0.0)
    assert good.finish_reason != "vetoed by a layer callback" and len(good.token_ids) >= 1
    ic = IntentClassifier.train(c, {"greet": safe, "noise": unsafe})
    assert ic.top(safe[2]) == "greet" and ic.top(unsafe[3]) == "noise"
    out, scores = ic.generate_with_intent(unsafe[3], max_tokens=3, temperature=0.0)      # read from the generation's own prefill
    assert max(scores, key=scores.get) == "noise" and len(out.token_ids) >= 1
    assert abs(scores["noise"] - ic.classify(unsafe[3])["noise"]) < 0.05
    tr = IntentTracker(ic)
    tr.update(safe[0]); tr.update(safe[1]); assert not tr.switched()
    tr.update(unsafe[0]); tr.update(unsafe[1]); tr.update(unsafe[2])
    assert tr.history[-1] == "noise" and abs(float(tr.state.pow(2).mean()) - 1.0) < 1e-3
    sg = StreamGuard.train(c, {"safe": safe, "unsafe": unsafe}, patience=1)
    out = list(sg.moderate_stream("", iter(["zzzz ", "qqqq ", "xxxx ", "zzzz "])))
    assert out[-1][1].risk == Risk.UNSAFE and len(out) <= 4
    assert sg.judge(safe[0]).risk == Risk.SAFE


def test_head_router_gatekeeper_and_late_fusion_rag():
    c = _client()
    hr = HeadRouter(c)
    p = hr.classify_multiway("is the sky blue? answer:", ["yes", "no", "maybe"])
    assert abs(sum(p.values()) - 1) < 1e-6 and hr.route("x", ["a", "b"]) in ("a", "b")
    assert 0.0 <= hr.classify_binary("q") <= 1.0
    assert hr.encode_to_layer(["abc"], 1).shape == (1, c._st().model.cfg.hidden_size)
    sg = SemanticGatekeeper(c, SemanticGatekeeperConfig(cooldown_tokens=2))
    k0 = sg.register("rust borrow checker lifetimes", SemanticLevel.L1_TOPIC, "lifetimes tie references to scopes")
    sg.register("french cooking butter sauce", SemanticLevel.L3_FACT)
    hit = sg.tap("rust borrow checker lifetimes")
    assert hit is not None and hit[0].key_id == k0 and hit[1] > 0.9 and hit[2] is not None
    assert sg.tap("rust borrow checker lifetimes") is None       # cooling down
    assert sg.injection_vector(k0).shape[0] == c._st().model.cfg.hidden_size

    class Sentinel:
        def in_code_context(self, text):
            return "```" in text
    sg2 = SemanticGatekeeper(c, sentinel=Sentinel())
    sg2.register("alpha beta", SemanticLevel.L1_TOPIC)
    assert sg2.tap("``` alpha beta") is None
    rag = LateFusionRag(c)
    docs = ["the cat sat on the mat", "stock markets fell sharply", "cats and kittens purr"]
    rag.index(docs)
    top, _, _ = rag.retrieve("the cat sat on the mat", top_k=1)
    assert top[0][0] == docs[0] and top[0][1] > 0.99
    v = rag.fusion_vector("cats purr", top_k=2)
    bus = ResidualBus(c._st().model.cfg.num_layers)
    chain = bus.chain(rag_vector=v, recall=["intent"])
    h = torch.zeros(3, v.shape[0])
    r = chain.run("pre", bus.ports["rag_inject"].layer, h)
    assert r.action == CallbackAction.REPLACE and torch.allclose(r.hidden[-1], v)
