"""Draft heads: the zero-parameter adapter (RMSNorm + shared lm_head), an EAGLE-style feature head, an MTP
(multi-token prediction) head, and the cache of drafts awaiting verification.

Reference parity: ``DraftAdapter``, ``EagleHead``, ``MtpHead``, ``SpeculationCache`` (src/speculative/*.rs);
MTP projection + argmax tail (src/arch/auto_graph_fragments/build_graph.inc.rs:2615-2655).
"""
from __future__ import annotations

from collections import OrderedDict
from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import torch

from .. import ops


def _rms(x, w, eps):
    return ops.rmsnorm(x, w, eps)


class DraftAdapter:
    """No new parameters: normalise an intermediate hidden state with the model's final norm and read it out
    through the shared lm_head (early-exit self-speculation)."""

    def __init__(self, final_norm: torch.Tensor, lm_head: torch.Tensor, eps: float = 1e-6):
        self.norm, self.lm_head, self.eps = final_norm, lm_head, eps

    def logits(self, hidden: torch.Tensor) -> torch.Tensor:
        return ops.gemm(_rms(hidden, self.norm, self.eps), self.lm_head, out_dtype=torch.float32)

    def draft_token(self, hidden: torch.Tensor) -> torch.Tensor:
        return self.logits(hidden).argmax(-1)


class EagleHead:
    """Predicts the next hidden FEATURE from [previous feature ; embedding of the sampled token] with one fused
    projection and a gated MLP, then reads tokens through the target's lm_head."""

    def __init__(self, hidden: int, embed: torch.Tensor, lm_head: torch.Tensor, final_norm: torch.Tensor, *, inter: int = 0,
                 seed: int = 0, dtype=None, eps: float = 1e-6):
        g = torch.Generator().manual_seed(seed)
        dt, dev = dtype or embed.dtype, embed.device
        inter = inter or 2 * hidden
        mk = lambda *s: (torch.randn(*s, generator=g) * 0.02).to(dev, dt)
        self.fc = mk(hidden, 2 * hidden)
        self.gate_up = mk(2 * inter, hidden)
        self.down = mk(hidden, inter)
        self.inter = inter
        self.embed, self.lm_head, self.norm, self.eps = embed, lm_head, final_norm, eps

    def step(self, feature: torch.Tensor, token: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        e = self.embed[token.long()].to(feature.dtype)
        h = ops.gemm(torch.cat([feature, e], -1).contiguous(), self.fc, out_dtype=feature.dtype)
        gu = ops.gemm(h, self.gate_up, out_dtype=feature.dtype)
        a = torch.nn.functional.silu(gu[:, :self.inter].float()) * gu[:, self.inter:].float()
        h = (h.float() + ops.gemm(a.to(feature.dtype), self.down, out_dtype=torch.float32)).to(feature.dtype)
        logits = ops.gemm(_rms(h, self.norm, self.eps), self.lm_head, out_dtype=torch.float32)
        return h, logits

    def draft(self, feature: torch.Tensor, token: torch.Tensor, depth: int) -> List[torch.Tensor]:
        out = []
        for _ in range(depth):
            feature, logits = self.step(feature, token)
            token = logits.argmax(-1)
            out.append(token)
        return out


class MtpHead:
    """DeepSeek-style multi-token prediction module for depth d: h' = proj([RMSNorm(h) ; RMSNorm(embed(t_{+d}))]),
    then the shared output head."""

    def __init__(self, hidden: int, embed: torch.Tensor, lm_head: torch.Tensor, *, seed: int = 0, dtype=None, eps: float = 1e-6):
        g = torch.Generator().manual_seed(seed)
        dt, dev = dtype or embed.dtype, embed.device
        self.h_norm = torch.ones(hidden, device=dev)
        self.e_norm = torch.ones(hidden, device=dev)
        self.out_norm = torch.ones(hidden, device=dev)
        self.proj = (torch.randn(hidden, 2 * hidden, generator=g) * 0.02).to(dev, dt)
        self.embed, self.lm_head, self.eps = embed, lm_head, eps

    def logits(self, hidden: torch.Tensor, next_token: torch.Tensor) -> torch.Tensor:
        e = self.embed[next_token.long()].to(hidden.dtype)
        x = torch.cat([_rms(hidden, self.h_norm, self.eps), _rms(e, self.e_norm, self.eps)], -1).contiguous()
        h = ops.gemm(x, self.proj, out_dtype=hidden.dtype)
        return ops.gemm(_rms(h, self.out_norm, self.eps), self.lm_head, out_dtype=torch.float32)


@dataclass
class DraftEntry:
    tokens: List[int]
    base_len: int
    step: int


class SpeculationCache:
    """Drafts by request id, bounded LRU."""

    def __init__(self, capacity: int = 1024):
        self.capacity = capacity
        self.d: "OrderedDict[int, DraftEntry]" = OrderedDict()

    def put(self, rid: int, tokens: List[int], base_len: int, step: int):
        self.d[rid] = DraftEntry(list(tokens), base_len, step)
        self.d.move_to_end(rid)
        while len(self.d) > self.capacity:
            self.d.popitem(last=False)

    def take(self, rid: int, base_len: int) -> Optional[DraftEntry]:
        e = self.d.pop(rid, None)
        return e if e is not None and e.base_len == base_len else None   # stale drafts are discarded
