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

    def as_callback(self):
        """The probe as a layer callback (the reference's form: the veto comes out of the forward itself, through
        callback slot 1, instead of re-encoding the text): after the probe layer the mean of the step's rows (the
        prompt's tokens in a prefill step, the new token's row in a decode step) is scored; an unsafe score vetoes."""
        from ..engine.callbacks import CallbackAction, CallbackResult, LayerCallback
        guard = self
        unsafe = self.probe.labels.index(self.unsafe_label)

        class _Probe(LayerCallback):
            priority = 20
            layers = [guard.layer]

            def post_layer(self, layer, hidden):
                p = guard.probe.probabilities(hidden.float().mean(0, keepdim=True).cpu())[0]
                info = {"guardrail_score": float(p[unsafe])}
                if float(p[unsafe]) > guard.threshold:
                    return CallbackResult(CallbackAction.VETO, info=info)
                return CallbackResult(info=info)
        return _Probe()

    def guarded_generate_in_flight(self, prompt: str, **kw):
        """Generate with the probe inside the forward: the request ends with finish reason ``vetoed by a layer
        callback`` as soon as a step's hidden state scores unsafe. Returns the client's response."""
        from ..engine.callbacks import CallbackChain
        b = self.client.generate(prompt).callbacks(CallbackChain([self.as_callback()]))
        for k, val in kw.items():
            b = getattr(b, k)(val)
        return b.generate()

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
