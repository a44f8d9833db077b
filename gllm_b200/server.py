"""HTTP front end over the serving loop: OpenAI-style completion, chat and embedding routes, server-sent-event
streaming, health and Prometheus metrics.

    python -m gllm_b200.server --model <id or path> [--host 127.0.0.1] [--port 8000] [--embedding-model <id>]

Every generation request goes to one ``engine.serving.ServingLoop``: requests of different connections share the
engine's batch step by step (continuous batching); a client that disconnects has its request cancelled. The reference
has no network front end (it is a library with a C ABI); this is an addition for deployment.
"""
import argparse
import json
import time
import uuid
from typing import List, Optional


def create_app(client, embedding_client=None):
    """A FastAPI application around ``client`` (a loaded chat model) and, optionally, an embedding model.
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
        if getattr(ac._loop.engine, "unhealthy", None):
            raise HTTPException(status_code=503, detail=f"engine unhealthy: {ac._loop.engine.unhealthy}")
        try:
            fut = ac.generate(prompt, stream=stream, **_params(body))
        except Exception as exc:
            raise HTTPException(status_code=400, detail=str(exc))
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
                for piece in fut.stream:
                    delta = {"delta": {"content": piece}} if chat else {"text": piece}
                    yield "data: " + json.dumps({"id": rid, "object": obj, "created": created, "model": model_name,
                                                 "choices": [{"index": 0, **delta, "finish_reason": None}]}) + "\n\n"
                r = fut.result()
                last = {"delta": {}} if chat else {"text": ""}
                yield "data: " + json.dumps({"id": rid, "object": obj, "created": created, "model": model_name,
                                             "choices": [{"index": 0, **last, "finish_reason": _finish(r.finish_reason)}],
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
    uvicorn.run(create_app(c, e), host=a.host, port=a.port, log_level="info")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
