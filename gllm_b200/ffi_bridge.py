"""Python side of the C ABI (``csrc/ffi/ffi.cpp``): builds a Client from (model id, options JSON) and returns
plain tuples that the shim copies into C structs."""
from __future__ import annotations

import json

import torch

_FINISH = {"eos": 1, "length": 2, "aborted": 3, "veto": 4}


class _Handle:
    def __init__(self, client):
        self.client = client

    def generate(self, prompt, max_tokens, temperature, top_k, top_p, thinking_budget=0):
        b = self.client.generate(prompt).max_tokens(int(max_tokens)).temperature(float(temperature))
        if top_k > 0:
            b = b.top_k(int(top_k))
        if top_p < 1.0:
            b = b.top_p(float(top_p))
        if thinking_budget > 0:          # 0: disabled, negative: unlimited (the reference's convention, src/ffi.rs:88)
            b = b.thinking_budget(int(thinking_budget))
        r = b.generate()
        return (r.text, [int(t) for t in r.token_ids], int(r.prompt_tokens), _FINISH.get(r.finish_reason, 0))

    def embed(self, text):
        out = self.client.embed([text]).normalize(True).generate()
        vec = out[0] if not hasattr(out, "embeddings") else out.embeddings[0]
        return [float(v) for v in (vec.tolist() if hasattr(vec, "tolist") else vec)]

    def rerank_score(self, query, document):
        res = self.client.rerank(query, [document]).generate()
        return float(res[0].score)

    def close(self):
        self.client.unload_model()


_KINDS = {0: "CHAT", 1: "EMBEDDING", 2: "RERANKER", 3: "CLASSIFIER"}    # the reference's kind_from_u32 (src/ffi.rs:30-37)


def create(model_id: str, kind: int = 0, options_json: str = "") -> _Handle:
    from .client import Client
    from .models.registry import ModelKind
    mk = getattr(ModelKind, _KINDS.get(int(kind), "CHAT"))
    from .models.config import preset
    from .models.weights import RandomWeights
    opts = json.loads(options_json) if options_json else {}
    device = opts.pop("device", "cuda:0" if torch.cuda.is_available() else "cpu")
    dtype = {"bf16": torch.bfloat16, "fp32": torch.float32, "fp16": torch.float16}[opts.pop("dtype", "bf16" if device != "cpu" else "fp32")]
    try:
        cfg = preset(model_id)
    except KeyError:
        cfg = None
    if cfg is not None:      # preset name: random-init weights of that architecture
        seed = int(opts.pop("seed", 0))
        client = Client.from_model(cfg, RandomWeights(cfg, "cpu" if device == "cpu" else device, dtype, seed=seed),
                                   kind=mk, device=device, dtype=dtype, **opts)
    else:
        ctor = {ModelKind.CHAT: Client.new_chat, ModelKind.EMBEDDING: Client.new_embedding,
                ModelKind.RERANKER: Client.new_reranker, ModelKind.CLASSIFIER: Client.new_classifier}[mk]
        client = ctor(model_id, device=device, **opts)
    return _Handle(client)
