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


class MtpExecutor:
    def __init__(self, depth: int, controller: AcceptanceController = None):
        self.depth = depth
        self.controller = controller or AcceptanceController(max_draft=depth)

    def active_depth(self) -> int:
        return min(self.depth, self.controller.draft_len())

    def verify(self, candidates: Sequence[int], target_argmax: Sequence[int]) -> MtpVerdict:
        """``target_argmax`` has len(candidates)+1 entries (after the main token, then after each candidate)."""
        n, nxt = verify_greedy(candidates, target_argmax)
        self.controller.update(n, len(candidates))
        return MtpVerdict(n, nxt, rollback_tokens=len(candidates) - n)
