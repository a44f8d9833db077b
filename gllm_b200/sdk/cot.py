"""Chain-of-thought reasoner: multi-step prompt orchestration over ``Client.generate`` (plan -> steps -> verify ->
answer, optional self-consistency voting).

Reference parity: src/cot_reasoner.rs (multi-step prompt orchestration over ``generate``).
"""
from __future__ import annotations

from collections import Counter
from dataclasses import dataclass, field
from typing import Callable, List, Optional


@dataclass
class CotConfig:
    max_steps: int = 4
    step_tokens: int = 96
    answer_tokens: int = 64
    temperature: float = 0.0
    samples: int = 1                       # > 1 = self-consistency majority vote
    thinking_budget: Optional[int] = None  # total tokens the steps may spend
    stop_marker: str = "FINAL:"


@dataclass
class CotTrace:
    question: str
    steps: List[str] = field(default_factory=list)
    answer: str = ""
    votes: Optional[Counter] = None
    tokens_used: int = 0


class CotReasoner:
    def __init__(self, client, cfg: CotConfig = CotConfig(), verifier: Optional[Callable[[str, str], bool]] = None):
        self.client, self.cfg, self.verifier = client, cfg, verifier

    def _gen(self, prompt: str, max_tokens: int, temperature: float):
        r = self.client.generate(prompt).max_tokens(max_tokens).temperature(temperature).generate()
        return r.text, len(r.token_ids)

    def _one(self, question: str, temperature: float) -> CotTrace:
        c = self.cfg
        tr = CotTrace(question)
        ctx = f"Question: {question}\nThink step by step.\n"
        for i in range(c.max_steps):
            budget = c.step_tokens if c.thinking_budget is None else min(c.step_tokens, c.thinking_budget - tr.tokens_used)
            if budget <= 0:
                break
            text, n = self._gen(ctx + f"Step {i + 1}:", budget, temperature)
            tr.tokens_used += n
            tr.steps.append(text.strip())
            ctx += f"Step {i + 1}: {text.strip()}\n"
            if c.stop_marker in text:
                break
        ans, n = self._gen(ctx + "Therefore, the answer is", c.answer_tokens, temperature)
        tr.tokens_used += n
        tr.answer = ans.split(c.stop_marker)[-1].strip()
        if self.verifier is not None and not self.verifier(question, tr.answer) and tr.tokens_used < (c.thinking_budget or 1 << 30):
            fix, n = self._gen(ctx + f"The answer '{tr.answer}' failed a check. Corrected answer:", c.answer_tokens, temperature)
            tr.tokens_used += n
            tr.steps.append("[revision]")
            tr.answer = fix.strip()
        return tr

    def reason(self, question: str) -> CotTrace:
        c = self.cfg
        if c.samples <= 1:
            return self._one(question, c.temperature)
        traces = [self._one(question, max(c.temperature, 0.7)) for _ in range(c.samples)]
        votes = Counter(t.answer for t in traces)
        best = votes.most_common(1)[0][0]
        out = next(t for t in traces if t.answer == best)
        out.votes = votes
        out.tokens_used = sum(t.tokens_used for t in traces)
        return out
