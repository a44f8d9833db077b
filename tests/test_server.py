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
