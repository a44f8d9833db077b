"""Weight blob: every packed tensor of a model in ONE contiguous allocation, 256-byte aligned, with an offset
table. One allocation means one upload / one peer mapping / one file section, TMA descriptors never straddle
allocations, and per-layer strides are constant for homogeneous layers.

Reference parity: ``pack_weights_from_graph`` -> contiguous blob in ``weight_layout`` order with per-layer
replication strides and mixed-quant offset tables (src/engine/mega_kernel/pack_observe.inc.rs:116-735).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import torch

ALIGN = 256


@dataclass
class BlobEntry:
    name: str
    offset: int
    nbytes: int
    shape: Tuple[int, ...]
    dtype: torch.dtype


class WeightBlob:
    def __init__(self, entries: List[BlobEntry], data: torch.Tensor):
        self.entries = {e.name: e for e in entries}
        self.order = [e.name for e in entries]
        self.data = data

    @staticmethod
    def pack(tensors: Dict[str, torch.Tensor], device=None, order: Optional[List[str]] = None) -> "WeightBlob":
        order = order or list(tensors)
        entries, off = [], 0
        for n in order:
            t = tensors[n]
            nbytes = t.numel() * t.element_size()
            entries.append(BlobEntry(n, off, nbytes, tuple(t.shape), t.dtype))
            off = (off + nbytes + ALIGN - 1) // ALIGN * ALIGN
        dev = device if device is not None else next(iter(tensors.values())).device
        data = torch.zeros(max(off, ALIGN), dtype=torch.uint8, device=dev)
        for e in entries:
            data[e.offset:e.offset + e.nbytes].copy_(tensors[e.name].contiguous().reshape(-1).view(torch.uint8))
        return WeightBlob(entries, data)

    def view(self, name: str) -> torch.Tensor:
        e = self.entries[name]
        return self.data[e.offset:e.offset + e.nbytes].view(e.dtype).view(*e.shape)

    def layer_stride(self, prefix_a: str, prefix_b: str) -> Optional[int]:
        """Constant byte distance between the tensors of two layers, or None when the layers differ in layout."""
        a = {n[len(prefix_a):]: e for n, e in self.entries.items() if n.startswith(prefix_a)}
        b = {n[len(prefix_b):]: e for n, e in self.entries.items() if n.startswith(prefix_b)}
        if not a or a.keys() != b.keys():
            return None
        d = {b[k].offset - a[k].offset for k in a}
        return d.pop() if len(d) == 1 else None

    def total_bytes(self) -> int:
        return int(self.data.numel())

    def offset_table(self) -> List[Tuple[str, int, int]]:
        return [(n, self.entries[n].offset, self.entries[n].nbytes) for n in self.order]
