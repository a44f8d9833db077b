"""Weight placement over tiers (L1 device, L2 pinned host, L3 memory-mapped file) and page compression of cold
weights.

Reference parity: src/loader/weight_tier.rs (L1 device / L2 host / L3 mmap placement),
src/loader/weight_compress.rs (LZ4 / zstd page compression; here zlib, the codecs in this image).
"""
from __future__ import annotations

import zlib
from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import torch


@dataclass
class TierPlacement:
    name: str
    bytes: int
    tier: int           # 1 device, 2 pinned host, 3 mmap
    reason: str = ""


def plan_weight_tiers(sizes: Dict[str, int], device_budget: int, host_budget: int,
                      always_resident=("embed_tokens", "lm_head", "norm", "router", "attn", "q_proj", "k_proj", "v_proj",
                                       "o_proj")) -> List[TierPlacement]:
    """Attention / norms / router / embeddings always stay on the device (every token needs them); expert and
    dense FFN weights fill what is left, largest layers index last (deep layers are reached last, so a prefetch has
    the most time to hide)."""
    out, dev, host = [], 0, 0
    def hot(n):
        return any(k in n for k in always_resident)
    for n in sorted(sizes, key=lambda n: (not hot(n), n)):
        b = sizes[n]
        if hot(n) or dev + b <= device_budget:
            out.append(TierPlacement(n, b, 1, "always resident" if hot(n) else "fits"))
            dev += b
        elif host + b <= host_budget:
            out.append(TierPlacement(n, b, 2, "device budget exhausted"))
            host += b
        else:
            out.append(TierPlacement(n, b, 3, "host budget exhausted"))
    return out


PAGE = 1 << 20


def compress_tensor(t: torch.Tensor, level: int = 3) -> Tuple[List[bytes], dict]:
    """Independent 1 MiB pages so that a page fault decompresses only what it needs."""
    raw = t.contiguous().view(torch.uint8).reshape(-1).numpy().tobytes()
    pages = [zlib.compress(raw[i:i + PAGE], level) for i in range(0, len(raw), PAGE)]
    meta = {"shape": tuple(t.shape), "dtype": str(t.dtype).replace("torch.", ""), "bytes": len(raw),
            "compressed": sum(len(p) for p in pages)}
    return pages, meta


def decompress_tensor(pages: List[bytes], meta: dict, page_range: Optional[range] = None) -> torch.Tensor:
    if page_range is not None:
        raw = b"".join(zlib.decompress(pages[i]) for i in page_range)
        return torch.frombuffer(bytearray(raw), dtype=torch.uint8)
    raw = b"".join(zlib.decompress(p) for p in pages)
    return torch.frombuffer(bytearray(raw), dtype=getattr(torch, meta["dtype"])).reshape(meta["shape"])
