"""Client surface on CPU with synthetic tiny models: generate / stream / hooks / sessions / batch / embed / rerank / classify."""
import torch

from gllm_b200.client import AsyncClient, Client, GllmError, InvalidModelTypeError, NoModelLoadedError
from gllm_b200.engine.batch import GenerateRequest
from gllm_b200.generation import GenerationHook, HookDecision, split_thinking_content
from gllm_b200.models.config import preset
from gllm_b200.models.registry import ModelKind
from gllm_b200.models.weights import RandomWeights
import pytest


def _chat():
    cfg = preset("tiny-qwen3")
    return Client.from_model(cfg, RandomWeights(cfg, "cpu", torch.float32, seed=3), device="cpu", dtype=torch.float32,
                             max_num_seqs=4, max_model_len=256, max_batch_tokens=64)


def test_generate_defaults_greedy_determinism_and_stream():
    c = _chat()
    b = c.generate("hello")
    assert (b._max_tokens, b._temperature, b._top_k, b._top_p) == (256, 0.7, 0, 1.0)   # reference defaults
    r1 = c.generate("hello world").max_tokens(6).temperature(0.0).generate()
    r2 = c.generate("hello world").max_tokens(6).temperature(0.0).generate()
    assert r1.token_ids == r2.token_ids and len(r1.token_ids) <= 6 and r1.prompt_tokens == 11
    assert r2.cached_prefix_tokens == 0          # 11 tokens never fill a 16-token page
    pieces = list(c.generate("hello world").max_tokens(6).temperature(0.0).stream().generate())
    assert "".join(pieces) == r1.text
    sampled = c.generate("hello world").max_tokens(6).temperature(0.9).top_k(5).top_p(0.9).generate()
    assert len(sampled.token_ids) <= 6


def test_hooks_veto_and_terminate_and_length_guard():
    c = _chat()

    class StopAt(GenerationHook):
        def __init__(self, n, how):
            self.n, self.how = n, how

        def post_step(self, token_id, n_generated):
            return self.how if n_generated == self.n else HookDecision.CONTINUE
    full = c.generate("abc").max_tokens(8).temperature(0.0).generate()
    t = c.generate("abc").max_tokens(8).temperature(0.0).hook(StopAt(3, HookDecision.TERMINATE)).generate()
    v = c.generate("abc").max_tokens(8).temperature(0.0).hook(StopAt(3, HookDecision.VETO)).generate()
    assert t.token_ids == full.token_ids[:3] and t.finish_reason == "terminate"
    assert v.token_ids == full.token_ids[:2] and v.finish_reason == "veto"   # the vetoed token is dropped
    with pytest.raises(GllmError):
        c.generate("x" * 300).max_tokens(10).generate()


def test_generate_batch_matches_single_and_session_prefix_reuse():
    c = _chat()
    prompts = ["the quick brown fox jumps over the lazy dog " * 2, "short", "another prompt of medium length here"]
    singles = [c.generate(p).max_tokens(5).temperature(0.0).generate().token_ids for p in prompts]
    batch = c.generate_batch([GenerateRequest(prompt=p, max_tokens=5, temperature=0.0) for p in prompts])
    eos = c._st().tokenizer.eos_ids(c._st().model.cfg.eos_token_ids)
    strip = lambda t: t[:-1] if t and t[-1] in eos else t
    assert [strip(r.token_ids) for r in batch] == singles
    # second turn of a conversation re-uses the cached pages of the first
    first = c.generate(prompts[0]).max_tokens(4).temperature(0.0).session_id("s1").generate()
    second = c.generate(prompts[0] + " and more").max_tokens(4).temperature(0.0).session_id("s1").generate()
    assert second.cached_prefix_tokens >= 64 and first.token_ids


def test_embed_rerank_classify_with_encoder():
    cfg = preset("tiny-bert")
    cfg.num_labels = 3
    src = RandomWeights(cfg, "cpu", torch.float32, seed=5)

    class Enc:  # canonical names of an encoder checkpoint on top of the random generator
        shapes = {"position_embeddings": (512, 128), "token_type_embeddings": (2, 128), "embed_norm": (128,),
                  "embed_norm_bias": (128,), "classifier": (3, 128), "classifier_bias": (3,), "pooler": (128, 128),
                  "pooler_bias": (128,)}

        def has(self, n):
            base = n.split(".")[-1]
            return n in self.shapes or base in ("q_proj", "k_proj", "v_proj", "o_proj", "up_proj", "down_proj",
                                                "post_attn_norm", "post_ffn_norm", "embed_tokens") or base.endswith("_bias")

        def get(self, n):
            base = n.split(".")[-1]
            if n in self.shapes:
                return src._gen(n, self.shapes[n], ones=n.endswith("norm"))
            if base.endswith("_bias"):
                stem = base[:-5]
                dim = {"up_proj": 256, "post_attn_norm": 128, "post_ffn_norm": 128}.get(stem, 128)
                return src._gen(n, (dim,))
            if base in ("post_attn_norm", "post_ffn_norm"):
                return src._gen(n, (128,), ones=True)
            return src.get(n)
    c = Client.from_model(cfg, Enc(), kind=ModelKind.CLASSIFIER, device="cpu", dtype=torch.float32)
    e = c.embed(["hello", "a longer sentence for the encoder"]).generate()
    assert len(e) == 2 and len(e[0]) == 128 and abs(sum(x * x for x in e[0]) - 1.0) < 1e-4
    e64 = c.embed(["hello"]).dimension(64).generate()
    assert len(e64[0]) == 64 and abs(sum(x * x for x in e64[0]) - 1.0) < 1e-4
    raw = c.embed(["hello"]).normalize(False).generate()[0]
    assert abs(sum(x * x for x in raw) - 1.0) > 1e-3
    # batched encoding equals one-at-a-time encoding (flat varlen batch with bidirectional attention)
    one = c.embed(["a longer sentence for the encoder"]).generate()[0]
    assert max(abs(a - b) for a, b in zip(one, e[1])) < 1e-4
    rr = c.rerank("query", ["doc one", "doc two", "doc three"]).top_n(2).generate()
    assert len(rr) == 2 and rr[0].score >= rr[1].score and rr[0].document.startswith("doc")
    cl = c.classify(["some text", "other"]).generate()
    assert len(cl) == 2 and 0 <= cl[0].label < 3 and abs(sum(cl[0].probabilities) - 1) < 1e-5
    with pytest.raises(InvalidModelTypeError):
        c.generate("x").generate()


def test_misc_api():
    with pytest.raises(NoModelLoadedError):
        Client().encode("x")
    c = _chat()
    assert c.decode(c.encode("round trip")) == "round trip"
    assert split_thinking_content("<think>plan</think> answer") == ("plan", "answer")
    assert split_thinking_content("plan</think>answer") == ("plan", "answer")
    ac = AsyncClient(c)
    f = ac.generate("hi", max_tokens=3, temperature=0.0)
    assert len(f.result(timeout=60).token_ids) <= 3
    ac.shutdown()
    d = c.diagnostics()
    assert d["backend"] == "cpu" and d["stats"]["decode_steps"] > 0
    s = c.score_tokens("hello", [1, 2, 3])
    assert len(s) == 3
    h = c.encode_to_layer(["hello there"], layer=0)
    assert h.shape == (1, 256)
    c.unload_model()
    with pytest.raises(NoModelLoadedError):
        c.generate("x").generate()


def test_kv_cache_plan_comes_from_the_decision_matrix():
    """Client.load picks the KV cache precision through the decision matrix: a cache that fits stays bf16, one that does
    not fit beside the weights asks for the low-precision variant (fp8 pages on a GPU)."""
    import torch
    from gllm_b200.client import Client, ClientConfig
    from gllm_b200.models.config import preset
    c = Client.__new__(Client)
    c.config = ClientConfig(max_num_seqs=8, max_model_len=1024)
    plan_kw = c._kv_cache_plan(preset("qwen3-8b"), torch.device("cpu"))
    assert plan_kw == {} and c.kv_plan["kv_cache_dtype"] == "bf16" and not c.kv_plan["variant"].kivi
    c.config = ClientConfig(max_num_seqs=4096, max_model_len=131072)      # 74 TB of bf16 KV: cannot fit
    c._kv_cache_plan(preset("qwen3-8b"), torch.device("cpu"))
    assert c.kv_plan["variant"].kivi and c.kv_plan["bf16_bytes"] > 180 << 30


def test_weight_quant_plan_of_the_client():
    """``ClientConfig.weight_quant``: explicit block-scaled formats build the fused block-scaled model (here on CPU
    tensors through the fp32 restatements of the fused ops); ``auto`` reads the checkpoint's quantisation tags and only
    acts on a GPU; shapes that do not fit are refused by name."""
    import pytest
    import torch
    from gllm_b200.client import Client
    from gllm_b200.models.config import preset
    from gllm_b200.models.weights import RandomWeights
    cfg = preset("tiny-qwen3")
    cfg.hidden_size, cfg.num_heads, cfg.num_kv_heads, cfg.head_dim, cfg.intermediate_size = 256, 2, 2, 128, 512
    src = RandomWeights(cfg, "cpu", torch.float32, seed=2, std=0.05)
    c = Client.from_model(cfg, src, device="cpu", dtype=torch.float32, max_num_seqs=2, max_model_len=128,
                          max_batch_tokens=64, weight_quant="mxfp8")
    model = c._state.model
    assert model.bs_fmt == "mxfp8" and model.fused
    r = c.generate("hello world").max_tokens(3).temperature(0.0).generate()
    assert 1 <= len(r.token_ids) <= 3
    # auto: tags of a 4-bit checkpoint -> nvfp4 on a GPU, nothing on the CPU
    cfg.quant = "Q4_K+Q6_K"
    plain = Client.from_model(cfg, src, device="cpu", dtype=torch.float32, max_num_seqs=2, max_model_len=128,
                              max_batch_tokens=64, weight_quant="auto")
    assert plain._state.model.bs_fmt is None
    assert plain._weight_quant_plan(cfg, torch.device("cuda")) == "nvfp4"
    cfg.quant = "Q8_0"
    assert plain._weight_quant_plan(cfg, torch.device("cuda")) == "mxfp8"
    cfg.quant = ""
    assert plain._weight_quant_plan(cfg, torch.device("cuda")) is None
    small = preset("tiny-qwen3")
    small.head_dim, small.num_heads, small.num_kv_heads = 64, 4, 2      # not the head size of the fused layer
    with pytest.raises(ValueError, match="do not fit"):
        Client.from_model(small, RandomWeights(small, "cpu", torch.float32, seed=2), device="cpu", dtype=torch.float32,
                          max_num_seqs=2, max_model_len=128, max_batch_tokens=64, weight_quant="nvfp4")


def test_async_client_batches_concurrent_callers_through_the_serving_loop():
    """Continuous mode: requests submitted from several threads run in one engine batch (more than one running
    sequence per step), every future resolves to what the blocking client returns, a request can be cancelled, and a
    bad request fails its own future only."""
    import threading
    import torch
    from gllm_b200.client import AsyncClient, Client
    from gllm_b200.models.config import preset
    from gllm_b200.models.weights import RandomWeights
    cfg = preset("tiny-qwen3")
    src = RandomWeights(cfg, "cpu", torch.float32, seed=2, std=0.05)
    kw = dict(device="cpu", dtype=torch.float32, max_num_seqs=8, max_model_len=128, max_batch_tokens=128)
    prompts = [f"request number {i} says hello" for i in range(6)]
    blocking = Client.from_model(cfg, src, **kw)
    want = [blocking.generate(p).max_tokens(12).temperature(0.0).generate().token_ids for p in prompts]
    ac = AsyncClient(Client.from_model(cfg, src, **kw), continuous=True)
    futs = [None] * len(prompts)

    def caller(i):
        futs[i] = ac.generate(prompts[i], max_tokens=12, temperature=0.0)
    threads = [threading.Thread(target=caller, args=(i,)) for i in range(len(prompts))]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    got = [f.result(timeout=120).token_ids for f in futs]
    assert got == want
    assert ac._loop.stats["max_running"] > 1 and ac._loop.stats["finished"] == 6
    streamed = ac.generate(prompts[2], max_tokens=12, temperature=0.0, stream=True)
    other = ac.generate(prompts[3], max_tokens=12, temperature=0.0)
    pieces = list(streamed.stream)                      # text arrives while both requests share the batch
    assert "".join(pieces) == streamed.result(timeout=60).text and streamed.result().token_ids == want[2]
    assert other.result(timeout=60).token_ids == want[3] and other.stream is None
    slow = ac.generate(prompts[0], max_tokens=100, temperature=0.0)
    assert ac.cancel(slow, "client went away")
    r = slow.result(timeout=120)
    assert r.finish_reason == "client went away" and len(r.token_ids) < 100
    bad = ac.generate("x " * 400, max_tokens=50)               # longer than the model allows
    try:
        bad.result(timeout=60)
        raised = False
    except Exception:
        raised = True
    assert raised and ac.generate(prompts[1], max_tokens=3, temperature=0.0).result(timeout=60).token_ids == want[1][:3]
    ac.shutdown()


def test_stop_strings_cut_the_text_and_end_the_request_early():
    from gllm_b200.client import AsyncClient
    from gllm_b200.generation import HookDecision, StopStringHook
    h = StopStringHook(lambda ids: "".join(chr(97 + i) for i in ids), ["de", "zz"])
    assert [h.post_step(t, i + 1) for i, t in enumerate([0, 1, 2, 3])] == [HookDecision.CONTINUE] * 4 and not h.hit
    assert h.post_step(4, 5) == HookDecision.TERMINATE and h.hit and h.cut("abcde") == "abc"
    c = _chat()
    c._st().tokenizer.decode = lambda ids: "".join(chr(97 + (int(i) % 26)) for i in ids)     # one letter per token
    full = c.generate("hello there").max_tokens(10).temperature(0.0).generate()
    assert len(full.text) == len(full.token_ids) == 10 and full.finish_reason == "length"
    stop = full.text[4:6]
    at = full.text.find(stop)
    r = c.generate("hello there").max_tokens(10).temperature(0.0).stop(stop).generate()
    assert r.text == full.text[:at] and r.finish_reason == "stop" and len(r.token_ids) == at + 2
    assert c.generate("hello there").max_tokens(10).temperature(0.0).stop(["#"]).generate().text == full.text
    ac = AsyncClient(c, continuous=True)
    try:
        r2 = ac.generate("hello there", max_tokens=10, temperature=0.0, stop=[stop]).result(timeout=120)
        assert r2.text == r.text and r2.finish_reason == "stop"
    finally:
        ac.shutdown()
