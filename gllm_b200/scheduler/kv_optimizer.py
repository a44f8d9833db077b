"""Scheduler-side KV optimiser: page importance from epilogue telemetry, precision-tier decision, page
requantisation, system-prompt compression candidates.

Reference parity: src/scheduler/kv_optimizer.rs:14-18,55-940:
``score = 120 * (1 - entropy / 6.93) + 80 * [softmax_max > 0.8] + 30 * head_spread / 255 - 40 * (1 - delta_rho)``
clamped to 0-255; sink or score > 200 -> page locked FP16; tiers > 200 FP16, > 150 FP8, > 80 KIVI4, > 40 KIVI2,
> 15 Sparse, else Evicted; Conversation pipeline never below FP8; per-depth-third layer floors; only decode-phase
pages are requantised (src/engine/executor_step.rs:265-393).
"""
from __future__ import annotations

from typing import Optional

import torch

from ..kv_cache.header import PrecisionTier
from ..kv_cache.quant import fp8_dequantize_page, fp8_quantize_page, kivi_dequantize, kivi_quantize_page
from .types import KvPipeline


def importance_score(entropy: float, softmax_max: float, head_spread: int, delta_rho: float) -> int:
    s = 120.0 * (1.0 - entropy / 6.93) + (80.0 if softmax_max > 0.8 else 0.0) + 30.0 * head_spread / 255.0 \
        - 40.0 * (1.0 - delta_rho)
    return int(max(0.0, min(255.0, s)))


def is_sink_page(score: int, has_sink_token: bool) -> bool:
    return has_sink_token or score > 200


LAYER_FLOORS = (PrecisionTier.FP8, PrecisionTier.KIVI4, PrecisionTier.KIVI2)   # first / middle / last third


def decide_tier(score: int, pipeline: KvPipeline = KvPipeline.WORKING, layer: Optional[int] = None,
                num_layers: Optional[int] = None, sink: bool = False) -> PrecisionTier:
    if sink or score > 200:
        t = PrecisionTier.FP16
    elif score > 150:
        t = PrecisionTier.FP8
    elif score > 80:
        t = PrecisionTier.KIVI4
    elif score > 40:
        t = PrecisionTier.KIVI2
    elif score > 15:
        t = PrecisionTier.SPARSE
    else:
        t = PrecisionTier.EVICTED
    if pipeline == KvPipeline.CONVERSATION and t > PrecisionTier.FP8:
        t = PrecisionTier.FP8
    if layer is not None and num_layers:
        floor = LAYER_FLOORS[min(2, 3 * layer // num_layers)]
        if pipeline == KvPipeline.WORKING and PrecisionTier.EVICTED > t > floor:
            t = floor
    return t


def requantize_page(k: torch.Tensor, v: torch.Tensor, tier: PrecisionTier):
    """Round-trip a page's K/V [tokens, D] through ``tier``'s representation. Returns (k, v, payload_bytes)."""
    if tier == PrecisionTier.FP16:
        return k, v, 2 * k.numel() * 2
    if tier == PrecisionTier.FP8:
        (kq, ks), (vq, vs) = fp8_quantize_page(k), fp8_quantize_page(v)
        return fp8_dequantize_page(kq, ks, k.dtype), fp8_dequantize_page(vq, vs, v.dtype), 2 * k.numel() + 8
    if tier in (PrecisionTier.KIVI4, PrecisionTier.KIVI2):
        p = kivi_quantize_page(k, v, bits=4 if tier == PrecisionTier.KIVI4 else 2)
        kd, vd = kivi_dequantize(p)
        return kd.to(k.dtype), vd.to(v.dtype), p.packed_bytes()
    if tier == PrecisionTier.SPARSE:   # keep the largest eighth of the entries
        def sp(x):
            kth = max(1, x.numel() // 8)
            thr = x.abs().flatten().topk(kth).values[-1]
            return torch.where(x.abs() >= thr, x, torch.zeros_like(x))
        return sp(k), sp(v), 2 * (k.numel() // 8) * 3
    return torch.zeros_like(k), torch.zeros_like(v), 0
