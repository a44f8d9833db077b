"""Decision matrix over KV optimisations: 16 variants = {KIVI, KVTuner, MUSTAFAR sparsity, ChunkKV} on/off,
chosen from a hardware profile and composed per page.

Reference parity: src/kv_cache/kv_optimizer/*.inc.rs.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List

from .header import PrecisionTier


@dataclass(frozen=True)
class KvVariant:
    kivi: bool = False          # low-bit asymmetric quantisation
    kvtuner: bool = False       # per-layer sensitivity-tuned precision
    mustafar: bool = False      # unstructured sparsity of near-zero KV entries
    chunkkv: bool = False       # semantic-chunk granularity retention

    @property
    def index(self) -> int:
        return int(self.kivi) | int(self.kvtuner) << 1 | int(self.mustafar) << 2 | int(self.chunkkv) << 3

    @staticmethod
    def from_index(i: int) -> "KvVariant":
        return KvVariant(bool(i & 1), bool(i & 2), bool(i & 4), bool(i & 8))

    def expected_bytes_ratio(self) -> float:
        r = 1.0
        if self.kivi:
            r *= 0.28
        if self.kvtuner:
            r *= 0.85
        if self.mustafar:
            r *= 0.6
        if self.chunkkv:
            r *= 0.75
        return r


ALL_VARIANTS: List[KvVariant] = [KvVariant.from_index(i) for i in range(16)]


@dataclass
class HardwareProfile:
    hbm_bytes: int = 180 << 30
    hbm_gbps: float = 6500.0
    has_fp8_tensor: bool = True
    has_fp4_tensor: bool = True
    sm_count: int = 148


class KvDecisionMatrix:
    def __init__(self, hw: HardwareProfile = HardwareProfile()):
        self.hw = hw

    def choose(self, kv_bytes_needed: int, weight_bytes: int, long_context: bool, latency_sensitive: bool) -> KvVariant:
        """Cheapest variant whose expected footprint fits what is left of HBM; nothing when everything fits."""
        free = self.hw.hbm_bytes * 0.92 - weight_bytes
        if kv_bytes_needed <= free:
            return KvVariant()
        ranked = sorted(ALL_VARIANTS[1:], key=lambda v: (bin(v.index).count("1"), v.expected_bytes_ratio()))
        for v in ranked:
            if latency_sensitive and v.mustafar:
                continue        # sparse gather costs decode latency
            if not long_context and v.chunkkv:
                continue
            if kv_bytes_needed * v.expected_bytes_ratio() <= free:
                return v
        return KvVariant(True, True, not latency_sensitive, long_context)

    @staticmethod
    def page_tier(variant: KvVariant, importance: int, layer_frac: float) -> PrecisionTier:
        """Compose the per-page precision from the variant, the page's importance (0-255) and the layer depth."""
        if not variant.kivi:
            return PrecisionTier.FP16 if importance > 15 or not variant.mustafar else PrecisionTier.SPARSE
        tier = PrecisionTier.FP16 if importance > 200 else PrecisionTier.FP8 if importance > 150 else \
            PrecisionTier.KIVI4 if importance > 80 else PrecisionTier.KIVI2
        if variant.kvtuner and layer_frac < 1 / 3 and tier > PrecisionTier.KIVI4:
            tier = PrecisionTier.KIVI4   # early layers are the sensitive ones
        return tier
