"""TurboQuant runtime: orchestrates rotation + low-bit quantisation of KV pages with FP16 attention sinks.

Reference parity: src/kv_cache/turboquant.rs:31-450; defaults (enabled only when some weight is quantised;
4-bit, 4 sink tokens kept FP16, FWHT on, deterministic rounding, dual-track off):
src/engine/executor_builder.rs:236-251.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional, Tuple

import torch

from .header import PrecisionTier
from .quant import KiviPage, kivi_dequantize, kivi_quantize_page


@dataclass
class TurboQuantConfig:
    enabled: bool = False
    bits: int = 4
    sink_tokens: int = 4
    use_fwht: bool = True
    stochastic_rounding: bool = False
    dual_track: bool = False

    @staticmethod
    def default_for(any_weight_quantised: bool) -> "TurboQuantConfig":
        return TurboQuantConfig(enabled=any_weight_quantised)


class TurboQuantRuntime:
    def __init__(self, cfg: TurboQuantConfig):
        self.cfg = cfg
        self.pages: Dict[Tuple[int, int, int], Tuple[KiviPage, Optional[torch.Tensor], Optional[torch.Tensor]]] = {}
        self.stats = {"pages": 0, "bytes_before": 0, "bytes_after": 0}

    def tier(self) -> PrecisionTier:
        return PrecisionTier.KIVI4 if self.cfg.bits >= 4 else PrecisionTier.KIVI2

    def compress(self, key, k: torch.Tensor, v: torch.Tensor, first_token_index: int = 0):
        """k, v: [tokens, D] of one (page, layer, head). Tokens that are global sinks stay in 16 bit."""
        if not self.cfg.enabled:
            return None
        n_sink = max(0, min(k.shape[0], self.cfg.sink_tokens - first_token_index))
        sink_k = k[:n_sink].clone() if n_sink else None
        sink_v = v[:n_sink].clone() if n_sink else None
        page = kivi_quantize_page(k, v, bits=self.cfg.bits, rotate=self.cfg.use_fwht and (k.shape[-1] & (k.shape[-1] - 1)) == 0,
                                  stochastic=self.cfg.stochastic_rounding)
        self.pages[key] = (page, sink_k, sink_v)
        self.stats["pages"] += 1
        self.stats["bytes_before"] += 2 * k.numel() * 2
        self.stats["bytes_after"] += page.packed_bytes() + (0 if sink_k is None else 2 * sink_k.numel() * 2)
        return page

    def decompress(self, key, dtype=torch.bfloat16):
        page, sink_k, sink_v = self.pages[key]
        k, v = kivi_dequantize(page)
        if sink_k is not None:
            k[:sink_k.shape[0]] = sink_k.float()
            v[:sink_v.shape[0]] = sink_v.float()
        return k.to(dtype), v.to(dtype)

    def compression_ratio(self) -> float:
        return self.stats["bytes_before"] / max(self.stats["bytes_after"], 1)
