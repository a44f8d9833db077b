"""Stream guard: a per-token moderation head over the backbone's last hidden state, evaluated while the tokens
stream (Safe / Controversial / Unsafe with a category).

Reference parity: src/qwen3_guard.rs (per-token moderation head on a qwen3 backbone).
"""
from __future__ import annotations

import enum
from dataclasses import dataclass
from typing import Iterator, List, Optional, Sequence, Tuple

import torch

from .probes import LinearProbe


class Risk(enum.Enum):
    SAFE = "safe"
    CONTROVERSIAL = "controversial"
    UNSAFE = "unsafe"


@dataclass
class TokenVerdict:
    index: int
    risk: Risk
    confidence: float


class StreamGuard:
    def __init__(self, client, probe: LinearProbe, layer: Optional[int] = None, patience: int = 2):
        self.client, self.probe, self.patience = client, probe, patience
        self.layer = layer if layer is not None else client._st().model.cfg.num_layers - 1

    @staticmethod
    def train(client, examples: dict, **kw) -> "StreamGuard":
        labels = [r.value for r in Risk if r.value in examples]
        layer = kw.pop("layer", None)
        layer = layer if layer is not None else client._st().model.cfg.num_layers - 1
        texts = [t for l in labels for t in examples[l]]
        y = torch.tensor([i for i, l in enumerate(labels) for _ in examples[l]])
        x = client.encode_to_layer(texts, layer, "last")
        return StreamGuard(client, LinearProbe.fit(x, y, labels), layer, **kw)

    def judge(self, text: str, index: int = 0) -> TokenVerdict:
        h = self.client.encode_to_layer([text], self.layer, "last")
        p = self.probe.probabilities(h)[0]
        i = int(p.argmax())
        return TokenVerdict(index, Risk(self.probe.labels[i]), float(p[i]))

    def moderate_stream(self, prompt: str, pieces: Iterator[str]) -> Iterator[Tuple[str, TokenVerdict]]:
        """Yields (piece, verdict); stops after ``patience`` consecutive unsafe verdicts."""
        text, bad = prompt, 0
        for i, piece in enumerate(pieces):
            text += piece
            v = self.judge(text, i)
            bad = bad + 1 if v.risk == Risk.UNSAFE else 0
            yield piece, v
            if bad >= self.patience:
                return
