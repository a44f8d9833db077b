"""Late-fusion RAG on the residual stream, the residual bus (named injection / recall ports) and early exit.

Reference parity: src/rag.rs:7-50 (late-fusion RAG), src/routing.rs (residual bus ports), src/early_exit.rs
(cosine / delta-rho exit); port layers (src/engine/executor_builder.rs:9-13,287-304).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import torch

from ..engine.callbacks import CallbackChain, EarlyExitCallback, MidLayerEncodeCallback, RagInjectCallback, port_layers


@dataclass
class Port:
    name: str
    layer: int
    direction: str            # "inject" | "recall"


class ResidualBus:
    def __init__(self, num_layers: int):
        self.num_layers = num_layers
        p = port_layers(num_layers)
        self.ports: Dict[str, Port] = {
            "rag_inject": Port("rag_inject", p["rag_inject"], "inject"),
            "early_exit": Port("early_exit", p["early_exit"], "recall"),
            "intent": Port("intent", p["intent"], "recall"),
            "guardrail": Port("guardrail", p["guardrail"], "recall"),
        }

    def chain(self, *, rag_vector: Optional[torch.Tensor] = None, rag_scale: float = 1.0, early_exit: bool = False,
              recall: Sequence[str] = ()) -> CallbackChain:
        cbs = []
        if rag_vector is not None:
            cbs.append(RagInjectCallback(self.ports["rag_inject"].layer, rag_vector, rag_scale))
        if early_exit:
            cbs.append(EarlyExitCallback(self.ports["early_exit"].layer))
        for name in recall:
            cbs.append(MidLayerEncodeCallback(self.ports[name].layer))
        return CallbackChain(cbs)


class LateFusionRag:
    """Documents are embedded once at the injection layer; at query time the best documents' vectors are mixed
    (similarity-weighted) into one residual injection instead of lengthening the prompt."""

    def __init__(self, client, layer: Optional[int] = None):
        self.client = client
        n = client._st().model.cfg.num_layers
        self.layer = layer if layer is not None else n // 2
        self.docs: List[str] = []
        self.vecs: Optional[torch.Tensor] = None

    def index(self, documents: Sequence[str]):
        self.docs = list(documents)
        self.vecs = self.client.encode_to_layer(self.docs, self.layer, "mean")

    def retrieve(self, query: str, top_k: int = 2):
        q = self.client.encode_to_layer([query], self.layer, "mean")[0]
        sims = torch.nn.functional.cosine_similarity(self.vecs, q[None], dim=-1)
        k = min(top_k, len(self.docs))
        val, idx = sims.topk(k)
        return [(self.docs[i], float(s)) for i, s in zip(idx.tolist(), val.tolist())], idx, val

    def fusion_vector(self, query: str, top_k: int = 2, temperature: float = 0.1) -> torch.Tensor:
        _, idx, val = self.retrieve(query, top_k)
        w = torch.softmax(val / temperature, 0)
        return (w[:, None] * self.vecs[idx]).sum(0)

    def generate(self, query: str, *, top_k: int = 2, scale: float = 1.0, **gen):
        """Answer ``query`` with the best documents fused into the residual stream at the injection layer (no longer
        prompt): ``gen`` are the generation settings (max_tokens, temperature, ...). Returns the client's response."""
        from ..engine.callbacks import CallbackChain, RagInjectCallback
        vec = self.fusion_vector(query, top_k)
        b = self.client.generate(query).callbacks(CallbackChain([RagInjectCallback(self.layer, vec, scale)]))
        for k, v in gen.items():
            b = getattr(b, k)(v)
        return b.generate()
