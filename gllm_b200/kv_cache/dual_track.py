"""Dual-track KV pool: a 3-4 bit main track plus a 1-bit sign residual track that can be dropped under pressure.

Reference parity: src/kv_cache/dual_track.rs:23-400.
"""
from __future__ import annotations

from typing import Dict

import torch

from .quant import apply_residual, kivi_dequantize, kivi_quantize_page, residual_sign_bits


class DualTrackPool:
    def __init__(self, main_bits: int = 4):
        self.main_bits = main_bits
        self.main: Dict[object, object] = {}
        self.residual: Dict[object, tuple] = {}

    def put(self, key, k: torch.Tensor, v: torch.Tensor):
        page = kivi_quantize_page(k, v, bits=self.main_bits)
        rk, rv = kivi_dequantize(page)
        self.main[key] = page
        self.residual[key] = (residual_sign_bits(k, rk), residual_sign_bits(v, rv))

    def get(self, key, use_residual: bool = True):
        k, v = kivi_dequantize(self.main[key])
        if use_residual and key in self.residual:
            (ks, km), (vs, vm) = self.residual[key]
            k, v = apply_residual(k, ks, km), apply_residual(v, vs, vm)
        return k, v

    def drop_residual(self, key=None) -> int:
        """Free the residual track (all pages, or one). Returns the bytes released."""
        keys = [key] if key is not None else list(self.residual)
        freed = 0
        for kk in keys:
            r = self.residual.pop(kk, None)
            if r is not None:
                freed += sum(s.numel() // 8 + m.numel() * 2 for s, m in r)
        return freed
