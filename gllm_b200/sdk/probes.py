"""Small trainable heads over hidden states shared by the SDKs (guardrail probe, intent classifier, stream
guard): closed-form ridge / softmax-regression fits so that a probe can be built from a handful of labelled
examples without an optimiser loop."""
from __future__ import annotations

from typing import List, Sequence

import torch


class LinearProbe:
    def __init__(self, weight: torch.Tensor, bias: torch.Tensor, labels: Sequence[str]):
        self.w, self.b, self.labels = weight, bias, list(labels)

    @staticmethod
    def fit(x: torch.Tensor, y: torch.Tensor, labels: Sequence[str], l2: float = 1e-2) -> "LinearProbe":
        """One-vs-rest ridge regression onto +-1 targets. x [n, d], y [n] int."""
        x = x.float()
        mu, sd = x.mean(0, keepdim=True), x.std(0, keepdim=True).clamp_min(1e-6)
        xn = (x - mu) / sd
        xa = torch.cat([xn, torch.ones(x.shape[0], 1)], 1)
        t = -torch.ones(x.shape[0], len(labels))
        t[torch.arange(x.shape[0]), y.long()] = 1.0
        a = xa.t() @ xa + l2 * torch.eye(xa.shape[1])
        sol = torch.linalg.solve(a, xa.t() @ t)                       # [d+1, C]
        w = sol[:-1] / sd.t()
        b = sol[-1] - (mu / sd) @ sol[:-1]
        return LinearProbe(w.t().contiguous(), b.reshape(-1), labels)

    def scores(self, x: torch.Tensor) -> torch.Tensor:
        return x.float() @ self.w.t() + self.b

    def predict(self, x: torch.Tensor) -> List[str]:
        return [self.labels[i] for i in self.scores(x).argmax(-1).tolist()]

    def probabilities(self, x: torch.Tensor) -> torch.Tensor:
        return torch.softmax(self.scores(x) * 4.0, -1)
