"""Guardrail: a probe classifier on a late-middle layer vetoes unsafe prompts / generations.

Reference parity: src/guardrail.rs (mid-layer probe classifier veto through the callback table;
src/client_fragments/client_impl.inc.rs:780-877); the probe layer defaults to L-2
(src/engine/executor_builder.rs:9-13).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence

import torch

from ..generation import GenerationHook, HookDecision
from .probes import LinearProbe


@dataclass
class GuardrailVerdict:
    allowed: bool
    label: str
    score: float


class Guardrail:
    def __init__(self, client, probe: LinearProbe, layer: Optional[int] = None, unsafe_label: str = "unsafe",
                 threshold: float = 0.5):
        self.client, self.probe, self.unsafe_label, self.threshold = client, probe, unsafe_label, threshold
        n = client._st().model.cfg.num_layers
        self.layer = layer if layer is not None else max(0, n - 2)

    @staticmethod
    def train(client, safe: Sequence[str], unsafe: Sequence[str], layer: Optional[int] = None, **kw) -> "Guardrail":
        n = client._st().model.cfg.num_layers
        layer = layer if layer is not None else max(0, n - 2)
        x = client.encode_to_layer(list(safe) + list(unsafe), layer, "mean")
        y = torch.tensor([0] * len(safe) + [1] * len(unsafe))
        return Guardrail(client, LinearProbe.fit(x, y, ["safe", "unsafe"]), layer, **kw)

    def check(self, text: str) -> GuardrailVerdict:
        h = self.client.encode_to_layer([text], self.layer, "mean")
        p = self.probe.probabilities(h)[0]
        i = self.probe.labels.index(self.unsafe_label)
        return GuardrailVerdict(float(p[i]) <= self.threshold, self.probe.labels[int(p.argmax())], float(p[i]))

    def guarded_generate(self, prompt: str, **kw):
        v = self.check(prompt)
        if not v.allowed:
            return None, v
        b = self.client.generate(prompt)
        for k, val in kw.items():
            b = getattr(b, k)(val)
        r = b.generate()
        out = self.check(prompt + r.text)
        return (r if out.allowed else None), out

    def hook(self, prompt: str, every: int = 16) -> GenerationHook:
        """A generation hook that re-checks the running text every ``every`` tokens and terminates on a veto."""
        guard = self

        class _Hook(GenerationHook):
            def __init__(self):
                self.ids: List[int] = []

            def post_step(self, token_id, n_generated):
                self.ids.append(token_id)
                if n_generated % every == 0:
                    text = prompt + guard.client.decode(self.ids)
                    if not guard.check(text).allowed:
                        return HookDecision.TERMINATE
                return HookDecision.CONTINUE
        return _Hook()
