"""Flat batch descriptors handed from the scheduler to the model.

Reference parity: ``BatchContext`` (flat header + per-sequence metadata, src/engine/batch_context.rs:21-167)
and ``GenerateRequest/GenerateResult`` (src/engine/batch_executor.rs:18-579). Here the descriptor is a
set of int32 device tensors: attention is the only op that needs per-token sequence lookup, every
GEMM / norm sees a flat M (SPEC/MD-ARCHIVE/20-BATCH-CONCURRENT-INFERENCE.md:18-48).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional

import torch


@dataclass
class ForwardBatch:
    token_ids: torch.Tensor          # [T] int32
    positions: torch.Tensor          # [T] int32
    slot_mapping: Optional[torch.Tensor]  # [T] int32 (page*16 + offset), -1 = do not write
    block_tables: torch.Tensor       # [S, max_blocks] int32
    ctx_lens: torch.Tensor           # [S] int32: KV tokens of each sequence after this step
    is_decode: bool = False          # one query token per sequence, T == S (slot-indexed)
    q_start: Optional[torch.Tensor] = None   # [S] int32 (prefill)
    q_len: Optional[torch.Tensor] = None     # [S] int32 (prefill)
    max_q_len: int = 1
    logits_rows: Optional[torch.Tensor] = None  # [R] int64 rows that need logits; None = all rows
    token_type_ids: Optional[torch.Tensor] = None
    causal: bool = True
    want_mtp: bool = False           # also run the model's multi-token-prediction heads on the logits rows
    cp: Optional[object] = None      # parallel.context_parallel.CpPrefill: exchange of KV pages before each attention

    @property
    def num_tokens(self) -> int:
        return int(self.token_ids.shape[0])


@dataclass
class GenerateRequest:
    """One request of ``generate_batch`` (defaults: src/generation.rs:447-461)."""
    prompt: str = ""
    prompt_token_ids: Optional[List[int]] = None
    max_tokens: int = 256
    temperature: float = 0.7
    top_k: int = 0
    top_p: float = 1.0
    session_id: Optional[str] = None
    stop_token_ids: Optional[List[int]] = None


@dataclass
class SequenceTelemetry:
    """Per-result telemetry (src/scheduler/telemetry.rs:7-31)."""
    prompt_tokens: int = 0
    generated_tokens: int = 0
    cached_prefix_tokens: int = 0
    preemptions: int = 0
    ttft_ms: float = 0.0
    tpot_ms: float = 0.0
    e2e_ms: float = 0.0


@dataclass
class GenerateResult:
    request_id: int
    token_ids: List[int]
    text: str = ""
    finish_reason: str = "length"
    telemetry: SequenceTelemetry = field(default_factory=SequenceTelemetry)
