"""64-byte per-page header, tier enums, page layout arithmetic and the front/back KV state.

Reference parity: ``KvPageHeader`` repr(C) 64 bytes with epilogue telemetry, quant meta, scheduler meta, codec,
storage tier, CRC16, compressed size, sequence id, logical index, last access (src/kv_cache/mod.rs:64-178);
``CompressionCodec`` (:183-194), ``StorageTier`` (:218-225), ``PrecisionTier`` (:295-310); ``KvPageLayout``
(:465-650); double buffer (:826-970). The header table is a numpy structured array so that it can be uploaded
to the device verbatim (pinned) and read by kernels as 64-byte records.
"""
from __future__ import annotations

import enum
from dataclasses import dataclass

import numpy as np


class CompressionCodec(enum.IntEnum):
    NONE = 0
    LZ4 = 1
    ZSTD = 2
    BITPACK_RLE = 3
    ZSTD_DICT = 4
    NVCOMP_ANS = 5


class StorageTier(enum.IntEnum):
    HBM = 0
    DRAM = 1
    NVME = 2
    REMOTE = 3


class PrecisionTier(enum.IntEnum):
    FP16 = 0
    FP8 = 1
    KIVI4 = 2
    KIVI2 = 3
    SPARSE = 4
    DICTIONARY = 5
    EVICTED = 6

    @property
    def bits(self) -> float:
        return {0: 16, 1: 8, 2: 4, 3: 2, 4: 1.0, 5: 1.0, 6: 0}[int(self)]


KV_PAGE_HEADER_DTYPE = np.dtype([
    ("page_id", "<u4"), ("ref_count", "<u2"), ("flags", "<u2"),
    # epilogue telemetry
    ("entropy", "<f2"), ("centroid", "<f2"), ("softmax_max", "<f2"), ("delta_rho", "<f2"),
    ("dead_ratio", "u1"), ("importance", "u1"), ("head_spread", "u1"), ("sink_mask_hi", "u1"),
    # quant meta
    ("sink_mask", "<u2"), ("channel_bitmap", "<u2"), ("k_scale_offset", "<u4"), ("precision_tier", "u1"),
    ("v_scale_e8", "u1"),
    # scheduler meta
    ("layer_mask", "<u2"), ("tier_age", "<u2"), ("pipeline", "u1"), ("deopt_flags", "u1"),
    ("codec", "u1"), ("storage_tier", "u1"), ("crc16", "<u2"), ("compressed_size", "<u4"),
    ("sequence_id", "<u8"), ("logical_index", "<u4"), ("last_access", "<u4"), ("_pad", "V4"),
])
assert KV_PAGE_HEADER_DTYPE.itemsize == 64, KV_PAGE_HEADER_DTYPE.itemsize


class KvPageHeaderTable:
    """One 64-byte header per physical page."""

    def __init__(self, num_pages: int):
        self.h = np.zeros(num_pages, dtype=KV_PAGE_HEADER_DTYPE)
        self.h["page_id"] = np.arange(num_pages, dtype=np.uint32)

    def __len__(self):
        return len(self.h)

    def bind(self, page: int, sequence_id: int, logical_index: int, now: int = 0, pipeline: int = 0):
        r = self.h[page]
        r["sequence_id"], r["logical_index"], r["last_access"], r["pipeline"] = sequence_id, logical_index, now, pipeline
        r["ref_count"] = 1
        r["precision_tier"], r["storage_tier"], r["codec"] = PrecisionTier.FP16, StorageTier.HBM, CompressionCodec.NONE

    def touch(self, page: int, now: int):
        self.h["last_access"][page] = now
        self.h["tier_age"][page] = 0

    def age_all(self):
        self.h["tier_age"] = np.minimum(self.h["tier_age"].astype(np.uint32) + 1, 65535).astype(np.uint16)

    def record_telemetry(self, page: int, entropy: float, softmax_max: float, delta_rho: float, dead_ratio: float = 0.0,
                         head_spread: int = 0, centroid: float = 0.0):
        r = self.h[page]
        r["entropy"], r["softmax_max"], r["delta_rho"], r["centroid"] = entropy, softmax_max, delta_rho, centroid
        r["dead_ratio"] = int(max(0.0, min(1.0, dead_ratio)) * 255)
        r["head_spread"] = int(max(0, min(255, head_spread)))

    def as_bytes(self) -> bytes:
        return self.h.tobytes()


@dataclass
class KvPageLayout:
    """Byte arithmetic of one page. Standard: [layer][K|V][kv_head][token][D]; MLA: [layer][token][d_c + d_rope]."""
    num_layers: int
    num_kv_heads: int
    head_dim: int
    page_size: int = 16
    elem_bytes: int = 2
    mla_dim: int = 0        # kv_lora_rank + rope dim; >0 selects the MLA layout
    header_bytes: int = 0   # 64 when headers are stored inline

    @property
    def layer_stride(self) -> int:
        if self.mla_dim:
            return self.page_size * self.mla_dim * self.elem_bytes
        return 2 * self.num_kv_heads * self.page_size * self.head_dim * self.elem_bytes

    @property
    def page_stride(self) -> int:
        return self.header_bytes + self.num_layers * self.layer_stride

    def k_offset(self, layer: int, head: int, token: int) -> int:
        if self.mla_dim:
            return self.header_bytes + layer * self.layer_stride + token * self.mla_dim * self.elem_bytes
        return self.header_bytes + layer * self.layer_stride + (head * self.page_size + token) * self.head_dim * self.elem_bytes

    def v_offset(self, layer: int, head: int, token: int) -> int:
        if self.mla_dim:
            return self.k_offset(layer, head, token)
        half = self.num_kv_heads * self.page_size * self.head_dim * self.elem_bytes
        return self.k_offset(layer, head, token) + half

    def pages_for(self, tokens: int) -> int:
        return (tokens + self.page_size - 1) // self.page_size

    def bytes_per_token(self) -> int:
        return self.num_layers * self.layer_stride // self.page_size

    def scale_bytes(self, tier: PrecisionTier) -> int:
        """Side storage for quantised tiers: K per channel (scale + zero), V per token."""
        if tier in (PrecisionTier.KIVI4, PrecisionTier.KIVI2):
            return self.num_layers * self.num_kv_heads * (self.head_dim * 4 + self.page_size * 4)
        if tier == PrecisionTier.FP8:
            return self.num_layers * self.num_kv_heads * 2 * 4
        return 0


class DoubleBufferedKvState:
    """Front (read by the running step) / back (being re-quantised or migrated) page sets; swap is O(1)."""

    def __init__(self):
        self.front, self.back = {}, {}
        self.generation = 0

    def stage(self, page: int, payload):
        self.back[page] = payload

    def publish(self):
        self.front.update(self.back)
        self.back = {}
        self.generation += 1

    def get(self, page: int):
        return self.front.get(page)
