"""MTP execution: the model emits its main token plus ``depth`` candidate tokens per step; the next step's full
logits verify the candidates; rejected ones roll the KV length back.

Reference parity: src/engine/mtp_executor.rs:15-425 (parse main + candidate tokens, verify vs full logits, EMA
acceptance controller, KV rollback instructions).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Sequence, Tuple

from .engine import AcceptanceController
from .verify import verify_greedy


@dataclass
class MtpStepOutput:
    main_token: int
    candidates: List[int]


def parse_step_tokens(flat: Sequence[int], depth: int) -> List[MtpStepOutput]:
    """The kernel writes [main, cand_1..cand_depth] per sequence, flat."""
    w = depth + 1
    return [MtpStepOutput(int(flat[i]), [int(x) for x in flat[i + 1:i + w]]) for i in range(0, len(flat), w)]


@dataclass
class MtpVerdict:
    accepted: int
    next_token: int
    rollback_tokens: int


class MtpController:
    """When the MTP heads are used and how deep, from the acceptance of their candidates.

    The policy and its numbers are the reference's (src/engine/mtp_executor.rs:159-285): an exponential average of the
    per-step acceptance (alpha 0.1, starting at 0.5); while active, three steps in a row under 0.3 switch the heads
    off; while off, five plain decode steps in a row (or steps whose acceptance is at least 0.5) switch them back on;
    the depth follows the average: above 0.8 the full depth, above 0.5 at most two, above 0.3 one, else none."""

    def __init__(self, max_depth: int, alpha: float = 0.1, disable_threshold: float = 0.3, enable_threshold: float = 0.5,
                 disable_patience: int = 3, enable_patience: int = 5):
        self.max_depth = max_depth
        self.alpha = min(1.0, max(0.01, alpha))
        self.disable_threshold, self.enable_threshold = disable_threshold, enable_threshold
        self.disable_patience, self.enable_patience = disable_patience, enable_patience
        self.ema = 0.5
        self.low_streak = self.stable_streak = 0
        self.enabled = True

    def update(self, accepted: int, proposed: int) -> bool:
        """One verify step (``proposed`` > 0) or one plain decode step (0, 0). Returns whether the heads are on."""
        rate = accepted / proposed if proposed > 0 else 0.0
        self.ema = self.alpha * rate + (1.0 - self.alpha) * self.ema
        if self.enabled:
            if rate < self.disable_threshold:
                self.low_streak += 1
                self.stable_streak = 0
            else:
                self.low_streak = 0
                self.stable_streak += 1
            if self.low_streak >= self.disable_patience:
                self.enabled, self.stable_streak = False, 0
        else:
            self.stable_streak = self.stable_streak + 1 if (rate >= self.enable_threshold or proposed == 0) else 0
            if self.stable_streak >= self.enable_patience:
                self.enabled, self.low_streak, self.stable_streak = True, 0, 0
        return self.enabled

    def draft_len(self) -> int:
        if not self.enabled:
            return 0
        if self.ema > 0.8:
            return self.max_depth
        if self.ema > 0.5:
            return min(self.max_depth, 2)
        return 1 if self.ema > 0.3 else 0


class MtpExecutor:
    def __init__(self, depth: int, controller=None):
        self.depth = depth
        self.controller = controller or MtpController(depth)

    def active_depth(self) -> int:
        return min(self.depth, self.controller.draft_len())

    def verify(self, candidates: Sequence[int], target_argmax: Sequence[int]) -> MtpVerdict:
        """``target_argmax`` has len(candidates)+1 entries (after the main token, then after each candidate)."""
        n, nxt = verify_greedy(candidates, target_argmax)
        self.controller.update(n, len(candidates))
        return MtpVerdict(n, nxt, rollback_tokens=len(candidates) - n)
