"""Speculative decoding state machine and a working prompt-lookup / self-drafting decoder on top of
``DecoderModel``.

Modes: STANDARD (separate draft model), EESD (early-exit self-drafting through the zero-parameter adapter),
SAGUARO (draft and verify on different GPUs), EAGLE (feature head), MTP (multi-token heads), NGRAM (prompt
lookup). ``should_speculate`` gates on batch size and on the acceptance EMA.

Reference parity: ``SpecDecodingState`` modes, ``should_speculate``, ``draft_phase`` / ``verify_phase``
(src/speculative/engine.rs:29-385); the acceptance controller (src/engine/mtp_executor.rs:15-425).
"""
from __future__ import annotations

import enum
from dataclasses import dataclass, field
from typing import Callable, List, Optional, Sequence

import torch

from ..engine.batch import ForwardBatch
from .tree import NgramIndex
from .verify import check_eqspec_invariants, verify_greedy


class SpecMode(enum.Enum):
    OFF = "off"
    STANDARD = "standard"
    EESD = "eesd"
    SAGUARO = "saguaro"
    EAGLE = "eagle"
    MTP = "mtp"
    NGRAM = "ngram"


@dataclass
class AcceptanceController:
    """EMA of the per-step acceptance rate drives the draft length (and switches speculation off when it does
    not pay)."""
    ema: float = 0.6
    alpha: float = 0.2
    min_draft: int = 1
    max_draft: int = 8
    off_below: float = 0.15

    def update(self, accepted: int, proposed: int):
        if proposed > 0:
            self.ema += self.alpha * (accepted / proposed - self.ema)

    def draft_len(self) -> int:
        if self.ema < self.off_below:
            return 0
        # expected accepted run for per-token acceptance a is a/(1-a): draft a little past it
        want = int(round(self.ema / max(1e-3, 1 - self.ema))) + 1
        return max(self.min_draft, min(self.max_draft, want))


@dataclass
class SpecDecodingState:
    mode: SpecMode = SpecMode.OFF
    max_batch_for_spec: int = 32
    controller: AcceptanceController = field(default_factory=AcceptanceController)
    steps: int = 0
    proposed: int = 0
    accepted: int = 0

    def should_speculate(self, batch_size: int, memory_pressure: float = 0.0) -> bool:
        """Speculation trades FLOPs for latency: only when the batch leaves the GPU memory-bound and KV has room."""
        if self.mode == SpecMode.OFF or batch_size > self.max_batch_for_spec or memory_pressure > 0.9:
            return False
        return self.controller.draft_len() > 0

    def record(self, proposed: int, accepted: int):
        self.steps += 1
        self.proposed += proposed
        self.accepted += accepted
        self.controller.update(accepted, proposed)

    @property
    def acceptance_rate(self) -> float:
        return self.accepted / max(self.proposed, 1)

    @property
    def tokens_per_step(self) -> float:
        return (self.accepted + self.steps) / max(self.steps, 1)


class SelfSpeculativeDecoder:
    """Single-sequence greedy decoding with drafts verified in ONE multi-token forward of the target.

    ``draft_fn(tokens, k) -> list[int]`` proposes up to k tokens; the default is prompt lookup (n-gram index over
    prompt + output). Rejected drafts leave stale KV entries past the committed length; they are overwritten by
    the next step (the block table is position-indexed), which is the rollback.
    """

    def __init__(self, model, num_pages: int = 64, draft_fn: Optional[Callable] = None, state: Optional[SpecDecodingState] = None):
        self.model = model
        self.kv = model.alloc_kv_cache(num_pages)
        self.num_pages = num_pages
        self.state = state or SpecDecodingState(SpecMode.NGRAM)
        self.ngram = NgramIndex()
        self.draft_fn = draft_fn or (lambda toks, k: (self.ngram.lookup(k) or [[]])[0])

    def _forward(self, tokens: Sequence[int], start: int) -> torch.Tensor:
        dev = self.model.device
        T = len(tokens)
        b = ForwardBatch(token_ids=torch.tensor(list(tokens), dtype=torch.int32, device=dev),
                         positions=torch.arange(start, start + T, dtype=torch.int32, device=dev),
                         slot_mapping=torch.arange(start, start + T, dtype=torch.int32, device=dev),
                         block_tables=torch.arange(self.num_pages, dtype=torch.int32, device=dev)[None],
                         ctx_lens=torch.tensor([start + T], dtype=torch.int32, device=dev),
                         q_start=torch.tensor([0], dtype=torch.int32, device=dev),
                         q_len=torch.tensor([T], dtype=torch.int32, device=dev), max_q_len=T)
        return self.model.forward(b, self.kv)[:, :self.model.cfg.vocab_size]

    def generate(self, prompt: Sequence[int], max_new_tokens: int, eos: Optional[int] = None) -> List[int]:
        toks = list(prompt)
        self.ngram.extend(toks)
        logits = self._forward(toks, 0)
        nxt = int(logits[-1].argmax())
        out: List[int] = []
        while len(out) < max_new_tokens:
            # `nxt` is decided but not yet in the KV cache
            k = self.state.controller.draft_len() if self.state.should_speculate(1) else 0
            k = min(k, max_new_tokens - len(out) - 1)
            self.ngram.extend([nxt])
            draft = list(self.draft_fn(toks + [nxt], k))[:k] if k > 0 else []
            before = list(toks)
            logits = self._forward([nxt] + draft, len(toks))
            arg = logits.argmax(-1).tolist()                  # arg[i]: target's token after nxt + draft[:i]
            n_acc, new_next = verify_greedy(draft, arg)
            toks = toks + [nxt] + draft[:n_acc]
            check_eqspec_invariants(before + [nxt], toks + [new_next], n_acc, new_next, draft)
            self.ngram.extend(draft[:n_acc])
            out.extend([nxt] + draft[:n_acc])
            if draft:
                self.state.record(len(draft), n_acc)
            nxt = new_next
            if eos is not None and eos in out:
                out = out[:out.index(eos) + 1]
                break
        return out[:max_new_tokens]
