"""HTTP front end over the serving loop: OpenAI-style completion, chat and embedding routes, server-sent-event
streaming, health and Prometheus metrics.

    python -m gllm_b200.server --model <id or path> [--host 127.0.0.1] [--port 8000] [--embedding-model <id>]
        [--reranker-model <id>] [--classifier-model <id>]

Every generation request goes to one ``engine.serving.ServingLoop``: requests of different connections share the
engine's batch step by step (continuous batching); a client that disconnects has its request cancelled. The reference
has no network front end (it is a library with a C ABI); this is an addition for deployment.
"""
import argparse
import json
import time
import uuid
from typing import List, Optional


class StopCutter:
    """Text filter for OpenAI-style ``stop`` strings over a stream of pieces: ``feed(piece)`` returns the text that is
    safe to show (a tail as long as the longest stop string minus one is held back, since a stop string may straddle
    two pieces) and sets ``hit`` once a stop string has appeared; nothing at or after it is ever returned."""

    def __init__(self, stops):
        self.stops = [s for s in stops if s]
        self.hold = max((len(s) for s in self.stops), default=1) - 1
        self.buf, self.hit = "", False

    def feed(self, piece: str) -> str:
        if self.hit:
            return ""
        self.buf += piece
        at = min((i for i in (self.buf.find(s) for s in self.stops) if i >= 0), default=-1)
        if at >= 0:
            out, self.buf, self.hit = self.buf[:at], "", True
            return out
        cut = len(self.buf) - self.hold
        if cut <= 0:
            return ""
        out, self.buf = self.buf[:cut], self.buf[cut:]
        return out

    def flush(self) -> str:
        out, self.buf = ("" if self.hit else self.buf), ""
        return out


def create_app(client, embedding_client=None, reranker_client=None, classifier_client=None):
    """A FastAPI application around ``client`` (a loaded chat model) and, optionally, an embedding, a reranker and a
    classifier model (``/v1/embeddings``, ``/v1/rerank``, ``/v1/classify``).
    (This module keeps real annotations, not strings: FastAPI reads the handlers' ``Request`` parameters from them.)"""
    from fastapi import FastAPI, HTTPException, Request
    from fastapi.responses import JSONResponse, PlainTextResponse, StreamingResponse

    from .client import AsyncClient
    from .utils.metrics import GLOBAL as METRICS

    app = FastAPI(title="gllm-b200")
    ac = AsyncClient(client, continuous=True)
    app.state.async_client = ac
    model_name = getattr(client._st(), "model_id", "model")

    def _params(body: dict) -> dict:
        p = {"max_tokens": int(body.get("max_tokens", 256)), "temperature": float(body.get("temperature", 0.7)),
             "top_p": float(body.get("top_p", 1.0)), "top_k": int(body.get("top_k", 0))}
        if body.get("session_id"):
            p["session_id"] = str(body["session_id"])
        return p

    def _chat_prompt(messages: List[dict]) -> str:
        tok = client._st().tokenizer
        tmpl = getattr(tok, "apply_chat_template", None)
        if callable(tmpl):
            try:
                return tmpl(messages)
            except Exception:
                pass
        return "".join(f"<|{m.get('role', 'user')}|>\n{m.get('content', '')}\n" for m in messages) + "<|assistant|>\n"

    def _usage(r) -> dict:
        return {"prompt_tokens": r.prompt_tokens, "completion_tokens": len(r.token_ids),
                "total_tokens": r.prompt_tokens + len(r.token_ids), "cached_prompt_tokens": r.cached_prefix_tokens}

    def _finish(reason: str) -> str:
        return {"eos": "stop", "length": "length"}.get(reason, reason)

    async def _run(request: Request, prompt: str, body: dict, chat: bool):
        import asyncio
        rid = ("chatcmpl-" if chat else "cmpl-") + uuid.uuid4().hex[:24]
        created = int(time.time())
        stream = bool(body.get("stream", False))
        stops = body.get("stop") or []
        stops = [stops] if isinstance(stops, str) else [str(x) for x in stops]
        if getattr(ac._loop.engine, "unhealthy", None):
            raise HTTPException(status_code=503, detail=f"engine unhealthy: {ac._loop.engine.unhealthy}")
        try:
            fut = ac.generate(prompt, stream=stream or bool(stops), **_params(body))
        except Exception as exc:
            raise HTTPException(status_code=400, detail=str(exc))
        cutter = StopCutter(stops) if stops else None

        def pieces():
            """The request's text pieces; with stop strings, cut at the first one (the request is cancelled there)."""
            for piece in fut.stream:
                if cutter is None:
                    yield piece
                    continue
                out = cutter.feed(piece)
                if out:
                    yield out
                if cutter.hit:
                    ac.cancel(fut, "stop")
                    return

        if not stream and cutter is not None:
            def collect():
                text = "".join(pieces())
                return text + cutter.flush()
            text = await asyncio.get_running_loop().run_in_executor(None, collect)
            try:
                r = fut.result()
            except Exception as exc:
                raise HTTPException(status_code=400, detail=str(exc))
            reason = "stop" if cutter.hit else _finish(r.finish_reason)
            choice = ({"index": 0, "message": {"role": "assistant", "content": text}, "finish_reason": reason}
                      if chat else {"index": 0, "text": text, "finish_reason": reason})
            return JSONResponse({"id": rid, "object": "chat.completion" if chat else "text_completion", "created": created,
                                 "model": model_name, "choices": [choice], "usage": _usage(r),
                                 "timing": {"ttft_ms": r.ttft_ms, "tpot_ms": r.tpot_ms}})
        if not stream:
            while not fut.done():
                if await request.is_disconnected():
                    ac.cancel(fut, "client disconnected")
                await asyncio.sleep(0.002)
            try:
                r = fut.result()
            except Exception as exc:
                raise HTTPException(status_code=400, detail=str(exc))
            choice = ({"index": 0, "message": {"role": "assistant", "content": r.text}, "finish_reason": _finish(r.finish_reason)}
                      if chat else {"index": 0, "text": r.text, "finish_reason": _finish(r.finish_reason)})
            return JSONResponse({"id": rid, "object": "chat.completion" if chat else "text_completion", "created": created,
                                 "model": model_name, "choices": [choice], "usage": _usage(r),
                                 "timing": {"ttft_ms": r.ttft_ms, "tpot_ms": r.tpot_ms}})

        def events():
            obj = "chat.completion.chunk" if chat else "text_completion"
            try:
                for piece in pieces():
                    delta = {"delta": {"content": piece}} if chat else {"text": piece}
                    yield "data: " + json.dumps({"id": rid, "object": obj, "created": created, "model": model_name,
                                                 "choices": [{"index": 0, **delta, "finish_reason": None}]}) + "\n\n"
                r = fut.result()
                tail = cutter.flush() if cutter is not None else ""
                last = {"delta": ({"content": tail} if tail else {})} if chat else {"text": tail}
                reason = "stop" if cutter is not None and cutter.hit else _finish(r.finish_reason)
                yield "data: " + json.dumps({"id": rid, "object": obj, "created": created, "model": model_name,
                                             "choices": [{"index": 0, **last, "finish_reason": reason}],
                                             "usage": _usage(r)}) + "\n\n"
            except Exception as exc:
                yield "data: " + json.dumps({"error": str(exc)}) + "\n\n"
            finally:
                if not fut.done():
                    ac.cancel(fut, "client disconnected")
            yield "data: [DONE]\n\n"
        return StreamingResponse(events(), media_type="text/event-stream")

    @app.post("/v1/completions")
    async def completions(request: Request):
        body = await request.json()
        prompt = body.get("prompt")
        if isinstance(prompt, list):
            prompt = prompt[0] if prompt else ""
        if not prompt:
            raise HTTPException(status_code=400, detail="prompt is required")
        return await _run(request, str(prompt), body, chat=False)

    @app.post("/v1/chat/completions")
    async def chat_completions(request: Request):
        body = await request.json()
        messages = body.get("messages")
        if not messages:
            raise HTTPException(status_code=400, detail="messages is required")
        return await _run(request, _chat_prompt(messages), body, chat=True)

    @app.post("/v1/embeddings")
    async def embeddings(request: Request):
        if embedding_client is None:
            raise HTTPException(status_code=400, detail="no embedding model is loaded")
        body = await request.json()
        texts = body.get("input")
        texts = [texts] if isinstance(texts, str) else list(texts or [])
        if not texts:
            raise HTTPException(status_code=400, detail="input is required")
        vecs = embedding_client.embed(texts).generate()
        data = [{"object": "embedding", "index": i, "embedding": [float(x) for x in v]} for i, v in enumerate(vecs)]
        return JSONResponse({"object": "list", "data": data, "model": getattr(embedding_client._st(), "model_id", "embedding")})

    @app.post("/v1/rerank")
    async def rerank(request: Request):
        if reranker_client is None:
            raise HTTPException(status_code=400, detail="no reranker model is loaded")
        body = await request.json()
        query, docs = body.get("query"), list(body.get("documents") or [])
        if not query or not docs:
            raise HTTPException(status_code=400, detail="query and documents are required")
        b = reranker_client.rerank(str(query), [str(d) for d in docs])
        if body.get("top_n"):
            b = b.top_n(int(body["top_n"]))
        results = [{"index": int(r.index), "relevance_score": float(r.score)} for r in b.generate()]
        return JSONResponse({"object": "list", "results": results,
                             "model": getattr(reranker_client._st(), "model_id", "reranker")})

    @app.post("/v1/classify")
    async def classify(request: Request):
        if classifier_client is None:
            raise HTTPException(status_code=400, detail="no classifier model is loaded")
        body = await request.json()
        texts = body.get("input")
        texts = [texts] if isinstance(texts, str) else list(texts or [])
        if not texts:
            raise HTTPException(status_code=400, detail="input is required")
        out = classifier_client.classify(texts).generate()
        data = [{"index": i, "label": int(r.label), "score": float(r.score), "probs": [float(p) for p in r.probabilities]}
                for i, r in enumerate(out)]
        return JSONResponse({"object": "list", "data": data,
                             "model": getattr(classifier_client._st(), "model_id", "classifier")})

    @app.get("/v1/models")
    async def models():
        return JSONResponse({"object": "list", "data": [{"id": model_name, "object": "model"}]})

    @app.get("/health")
    async def health():
        loop = ac._loop
        eng = loop.engine
        return JSONResponse({"status": "unhealthy" if getattr(eng, "unhealthy", None) else "ok", "running": int(eng.batcher.num_running),
                             "waiting": int(eng.batcher.num_waiting), "free_pages": int(eng.batcher.num_free_pages),
                             "loop": dict(loop.stats)})

    @app.get("/metrics")
    async def metrics():
        from prometheus_client import generate_latest
        return PlainTextResponse(generate_latest(METRICS.export_prometheus()).decode(), media_type="text/plain; version=0.0.4")

    @app.on_event("shutdown")
    def _shutdown():
        ac.shutdown()

    return app


def main(argv: Optional[List[str]] = None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--model", required=True)
    ap.add_argument("--embedding-model", default=None)
    ap.add_argument("--reranker-model", default=None)
    ap.add_argument("--classifier-model", default=None)
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--port", type=int, default=8000)
    ap.add_argument("--max-num-seqs", type=int, default=256)
    ap.add_argument("--max-model-len", type=int, default=4096)
    ap.add_argument("--weight-quant", default="bf16")
    a = ap.parse_args(argv)
    import uvicorn

    from .client import Client
    c = Client.builder().model(a.model).config(max_num_seqs=a.max_num_seqs, max_model_len=a.max_model_len,
                                               weight_quant=a.weight_quant).build()
    e = Client.new_embedding(a.embedding_model) if a.embedding_model else None
    r = Client.new_reranker(a.reranker_model) if a.reranker_model else None
    k = Client.new_classifier(a.classifier_model) if a.classifier_model else None
    uvicorn.run(create_app(c, e, r, k), host=a.host, port=a.port, log_level="info")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
