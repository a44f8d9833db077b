"""Head routing: classification by reading the generator's own output head at chosen vocabulary rows.

Reference parity: ``classify_binary / classify_multiway`` and ``encode_to_layer`` reusing the generator's lm_head
rows (src/head_routing.rs; src/client_fragments/client_impl.inc.rs:500-632).
"""
from __future__ import annotations

import math
from typing import Dict, List, Sequence


class HeadRouter:
    def __init__(self, client):
        self.client = client

    def _first_token(self, word: str) -> int:
        tok = self.client._st().tokenizer
        tid = tok.token_to_id(word) if hasattr(tok, "token_to_id") else None
        return tid if tid is not None else tok.encode(word, False)[0]

    def classify_multiway(self, prompt: str, options: Sequence[str]) -> Dict[str, float]:
        ids = [self._first_token(o) for o in options]
        logits = self.client.score_tokens(prompt, ids)
        m = max(logits)
        ex = [math.exp(l - m) for l in logits]
        s = sum(ex)
        return {o: e / s for o, e in zip(options, ex)}

    def classify_binary(self, prompt: str, positive: str = "yes", negative: str = "no") -> float:
        return self.classify_multiway(prompt, [positive, negative])[positive]

    def route(self, prompt: str, options: Sequence[str]) -> str:
        p = self.classify_multiway(prompt, options)
        return max(p, key=p.get)

    def encode_to_layer(self, texts: Sequence[str], layer: int, pooling: str = "mean"):
        return self.client.encode_to_layer(texts, layer, pooling)
