"""HTTP front end over the serving loop (FastAPI test client, tiny synthetic model on CPU)."""
import json

import pytest
import torch

fastapi = pytest.importorskip("fastapi")
pytest.importorskip("httpx")


def _app():
    from gllm_b200.client import Client
    from gllm_b200.models.config import preset
    from gllm_b200.models.weights import RandomWeights
    from gllm_b200.server import create_app
    cfg = preset("tiny-qwen3")
    c = Client.from_model(cfg, RandomWeights(cfg, "cpu", torch.float32, seed=2, std=0.05), device="cpu", dtype=torch.float32,
                          max_num_seqs=8, max_model_len=128, max_batch_tokens=128)
    return c, create_app(c)


def test_completion_chat_stream_health_and_metrics():
    from fastapi.testclient import TestClient
    c, app = _app()
    with TestClient(app) as http:
        r = http.post("/v1/completions", json={"prompt": "hello world", "max_tokens": 6, "temperature": 0.0})
        assert r.status_code == 200
        body = r.json()
        assert body["object"] == "text_completion" and body["usage"]["completion_tokens"] == 6
        assert body["choices"][0]["finish_reason"] == "length" and isinstance(body["choices"][0]["text"], str)
        r = http.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "hi"}], "max_tokens": 4,
                                                    "temperature": 0.0})
        assert r.status_code == 200 and r.json()["choices"][0]["message"]["role"] == "assistant"
        # streaming: server-sent events whose pieces add up to the text of the blocking call
        ref = http.post("/v1/completions", json={"prompt": "stream me", "max_tokens": 8, "temperature": 0.0}).json()
        pieces, finish = [], None
        with http.stream("POST", "/v1/completions", json={"prompt": "stream me", "max_tokens": 8, "temperature": 0.0,
                                                          "stream": True}) as resp:
            assert resp.status_code == 200
            for line in resp.iter_lines():
                if not line or not line.startswith("data: ") or line == "data: [DONE]":
                    continue
                ev = json.loads(line[6:])
                pieces.append(ev["choices"][0]["text"])
                finish = ev["choices"][0]["finish_reason"] or finish
        assert "".join(pieces) == ref["choices"][0]["text"] and finish == "length"
        assert http.post("/v1/completions", json={"max_tokens": 3}).status_code == 400
        assert http.post("/v1/completions", json={"prompt": "x " * 400, "max_tokens": 50}).status_code == 400   # too long
        assert http.post("/v1/embeddings", json={"input": "a"}).status_code == 400                             # none loaded
        h = http.get("/health").json()
        assert h["status"] == "ok" and h["loop"]["finished"] >= 4 and h["running"] == 0
        assert http.get("/v1/models").json()["data"][0]["object"] == "model"
        m = http.get("/metrics")
        assert m.status_code == 200 and "gllm_" in m.text
        # a device fault marks the engine unhealthy: the front end answers 503 and says why
        app.state.async_client._loop.engine.unhealthy = "device status 5 (timeout waiting for a peer)"
        r = http.post("/v1/completions", json={"prompt": "hello", "max_tokens": 2})
        assert r.status_code == 503 and "unhealthy" in r.json()["detail"]
        assert http.get("/health").json()["status"] == "unhealthy"
        app.state.async_client._loop.engine.unhealthy = None
        assert http.post("/v1/completions", json={"prompt": "hello", "max_tokens": 2, "temperature": 0.0}).status_code == 200


def test_stop_cutter_holds_back_a_straddling_stop_string():
    from gllm_b200.server import StopCutter
    c = StopCutter(["END", "\n\n"])
    out = [c.feed(p) for p in ("abc", "dE", "N", "D tail", "more")]
    assert "".join(out) == "abcd" and c.hit and c.flush() == ""
    c = StopCutter(["END"])
    shown = c.feed("hello E") + c.feed("N")
    assert shown == "hello " and not c.hit and shown + c.flush() == "hello EN"


def test_stop_strings_rerank_and_classify_routes():
    from types import SimpleNamespace as NS
    from fastapi.testclient import TestClient
    from gllm_b200.client import ClassifyResult, RerankResult
    from gllm_b200.server import create_app

    class Builder:
        def __init__(self, rows):
            self.rows = rows

        def top_n(self, n):
            return Builder(self.rows[:n])

        def generate(self):
            return self.rows

    class Aux:                                          # what the routes need of a reranker / classifier client
        def _st(self):
            return NS(model_id="aux")

        def rerank(self, q, docs):
            return Builder(sorted((RerankResult(i, float(len(d)), d) for i, d in enumerate(docs)), key=lambda r: -r.score))

        def classify(self, texts):
            return Builder([ClassifyResult(len(t) % 2, 0.75, [0.25, 0.75][::1 if len(t) % 2 else -1]) for t in texts])

    c, _ = _app()
    app = create_app(c, None, Aux(), Aux())
    with TestClient(app) as http:
        # the stop logic against a scripted stream (a random-weight model's text is not a stable fixture)
        ac, cancelled = app.state.async_client, []
        real_generate, real_cancel = ac.generate, ac.cancel

        def scripted(prompt, **kw):
            assert kw.get("stream") is True
            res = NS(text="abcdEND tail", token_ids=[1, 2, 3, 4], prompt_tokens=3, cached_prefix_tokens=0,
                     finish_reason="length", ttft_ms=1.0, tpot_ms=1.0)
            return NS(stream=iter(["abc", "dE", "ND", " tail"]), result=lambda: res, done=lambda: True)
        ac.generate, ac.cancel = scripted, lambda fut, reason="aborted": cancelled.append(reason)
        r = http.post("/v1/completions", json={"prompt": "p", "stop": "END"}).json()
        assert r["choices"][0]["text"] == "abcd" and r["choices"][0]["finish_reason"] == "stop" and cancelled == ["stop"]
        r = http.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "p"}], "stop": ["zz", "c"]}).json()
        assert r["choices"][0]["message"]["content"] == "ab" and r["choices"][0]["finish_reason"] == "stop"
        r = http.post("/v1/completions", json={"prompt": "p", "stop": "never"}).json()
        assert r["choices"][0]["text"] == "abcdEND tail" and r["choices"][0]["finish_reason"] == "length"
        pieces, finish = [], None
        with http.stream("POST", "/v1/completions", json={"prompt": "p", "stop": ["END"], "stream": True}) as resp:
            for line in resp.iter_lines():
                if line.startswith("data: ") and line != "data: [DONE]":
                    ev = json.loads(line[6:])
                    pieces.append(ev["choices"][0]["text"])
                    finish = ev["choices"][0]["finish_reason"] or finish
        assert "".join(pieces) == "abcd" and finish == "stop"
        ac.generate, ac.cancel = real_generate, real_cancel
        # through the engine: a stop string that never appears changes nothing
        r = http.post("/v1/completions", json={"prompt": "stop test prompt", "max_tokens": 12, "temperature": 0.0,
                                               "stop": "\x00never\x00"}).json()
        assert r["choices"][0]["finish_reason"] == "length" and r["usage"]["completion_tokens"] == 12
        rr = http.post("/v1/rerank", json={"query": "q", "documents": ["a", "ccc", "bb"], "top_n": 2}).json()
        assert [x["index"] for x in rr["results"]] == [1, 2] and rr["model"] == "aux"
        cl = http.post("/v1/classify", json={"input": ["ab", "abc"]}).json()
        assert [x["label"] for x in cl["data"]] == [0, 1] and abs(sum(cl["data"][0]["probs"]) - 1) < 1e-6
        assert http.post("/v1/rerank", json={"query": "q"}).status_code == 400
        assert http.get("/health").json()["running"] == 0
