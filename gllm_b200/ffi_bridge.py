"""Python side of the C ABI (``csrc/ffi/ffi.cpp``): builds a Client from (model id, options JSON) and returns
plain tuples that the shim copies into C structs."""
from __future__ import annotations

import json

import torch

_FINISH = {"eos": 1, "length": 2, "aborted": 3, "veto": 4}


class _Handle:
    def __init__(self, client):
        self.client = client

    def generate(self, prompt, max_tokens, temperature, top_k, top_p):
        b = self.client.generate(prompt).max_tokens(int(max_tokens)).temperature(float(temperature))
        if top_k > 0:
            b = b.top_k(int(top_k))
        if top_p < 1.0:
            b = b.top_p(float(top_p))
        r = b.generate()
        return (r.text, [int(t) for t in r.token_ids], int(r.prompt_tokens), _FINISH.get(r.finish_reason, 0))

    def close(self):
        self.client.unload_model()


def create(model_id: str, options_json: str = "") -> _Handle:
    from .client import Client
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
                                   device=device, dtype=dtype, **opts)
    else:
        client = Client.new_chat(model_id, device=device, **opts)
    return _Handle(client)
