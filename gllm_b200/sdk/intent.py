"""Intent classification from a mid-layer hidden state and a recurrent tracker over a conversation.

Reference parity: src/intent.rs, src/intent_tracker.rs (mid-layer hidden extraction + small classifier);
the pure-scalar tracker cell with sigmoid / silu / matvec / rmsnorm (src/arch/c1_v2_tracker.rs:512-560); the
intent port sits at 0.75 L (src/engine/executor_builder.rs:9-13).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import torch

from .probes import LinearProbe


class IntentClassifier:
    def __init__(self, client, probe: LinearProbe, layer: int):
        self.client, self.probe, self.layer = client, probe, layer

    @staticmethod
    def train(client, examples: Dict[str, Sequence[str]], layer: Optional[int] = None) -> "IntentClassifier":
        n = client._st().model.cfg.num_layers
        layer = layer if layer is not None else int(0.75 * n)
        labels = list(examples)
        texts = [t for l in labels for t in examples[l]]
        y = torch.tensor([i for i, l in enumerate(labels) for _ in examples[l]])
        x = client.encode_to_layer(texts, layer, "mean")
        return IntentClassifier(client, LinearProbe.fit(x, y, labels), layer)

    def hidden(self, text: str) -> torch.Tensor:
        return self.client.encode_to_layer([text], self.layer, "mean")[0]

    def classify(self, text: str) -> Dict[str, float]:
        p = self.probe.probabilities(self.hidden(text)[None])[0]
        return {l: float(v) for l, v in zip(self.probe.labels, p)}

    def top(self, text: str) -> str:
        c = self.classify(text)
        return max(c, key=c.get)

    def as_callback(self):
        """The classifier on the intent port of the residual bus (0.75 L): the prompt's intent is read from the prefill
        forward of the generation itself (mean of the prompt rows at the probe layer), no second encode. The result is
        left in ``callback.scores`` and in the model's ``callback_info["intent"]``."""
        from ..engine.callbacks import CallbackResult, LayerCallback
        clf = self

        class _Intent(LayerCallback):
            priority = 5
            layers = [clf.layer]
            scores: Optional[Dict[str, float]] = None

            def post_layer(self, layer, hidden):
                if hidden.shape[0] < 2 and self.scores is not None:
                    return CallbackResult()          # decode steps: the prompt's intent stands
                p = clf.probe.probabilities(hidden.float().mean(0, keepdim=True).cpu())[0]
                self.scores = {l: float(v) for l, v in zip(clf.probe.labels, p)}
                return CallbackResult(info={"intent": max(self.scores, key=self.scores.get)})
        return _Intent()

    def generate_with_intent(self, prompt: str, **gen):
        """(response, intent scores of the prompt) from one generation call."""
        from ..engine.callbacks import CallbackChain
        cb = self.as_callback()
        b = self.client.generate(prompt).callbacks(CallbackChain([cb]))
        for k, v in gen.items():
            b = getattr(b, k)(v)
        return b.generate(), cb.scores


def _rmsnorm(x, eps=1e-6):
    return x * torch.rsqrt(x.pow(2).mean() + eps)


class IntentTrackerCell:
    """Gated recurrent cell over per-turn hidden states:
    z = sigmoid(Wz [h; s]), c = silu(Wc [h; s]), s' = rmsnorm((1 - z) * s + z * c)."""

    def __init__(self, hidden: int, state: int = 64, seed: int = 0):
        g = torch.Generator().manual_seed(seed)
        self.wz = torch.randn(state, hidden + state, generator=g) / (hidden + state) ** 0.5
        self.wc = torch.randn(state, hidden + state, generator=g) / (hidden + state) ** 0.5
        self.state_dim = state

    def step(self, h: torch.Tensor, s: torch.Tensor) -> torch.Tensor:
        v = torch.cat([_rmsnorm(h.float()), s])
        z = torch.sigmoid(self.wz @ v)
        c = torch.nn.functional.silu(self.wc @ v)
        return _rmsnorm((1 - z) * s + z * c)


@dataclass
class IntentTracker:
    classifier: IntentClassifier
    cell: Optional[IntentTrackerCell] = None
    state: Optional[torch.Tensor] = None
    history: List[str] = field(default_factory=list)
    smoothing: float = 0.5
    belief: Dict[str, float] = field(default_factory=dict)

    def update(self, utterance: str) -> Dict[str, float]:
        h = self.classifier.hidden(utterance)
        if self.cell is None:
            self.cell = IntentTrackerCell(h.shape[0])
            self.state = torch.zeros(self.cell.state_dim)
        self.state = self.cell.step(h, self.state)
        now = self.classifier.classify(utterance)
        self.belief = {k: self.smoothing * self.belief.get(k, 1.0 / len(now)) + (1 - self.smoothing) * v for k, v in now.items()}
        self.history.append(max(self.belief, key=self.belief.get))
        return self.belief

    def switched(self) -> bool:
        return len(self.history) >= 2 and self.history[-1] != self.history[-2]
