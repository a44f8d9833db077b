"""SafeTensors: zero-copy memory-mapped reader (single file or sharded with ``model.safetensors.index.json``),
typed views, ``__metadata__`` access, and a writer.

Reference parity: ``loader/safetensors.rs:138-470`` — mmap, multi-shard, typed views, quantisation-group
detection (AWQ / GPTQ / MXFP4 / NVFP4 / FP8), ``gllm_config`` metadata. The format is implemented here
directly (8-byte little-endian header length, JSON header, raw little-endian data) instead of through the
``safetensors`` package so the loader has no hidden copies.
"""
from __future__ import annotations

import json
import mmap
import struct
from pathlib import Path
from typing import Any, Dict, Iterable, List, Optional

import numpy as np
import torch

_DTYPES = {
    "F64": (torch.float64, 8), "F32": (torch.float32, 4), "F16": (torch.float16, 2), "BF16": (torch.bfloat16, 2),
    "I64": (torch.int64, 8), "I32": (torch.int32, 4), "I16": (torch.int16, 2), "I8": (torch.int8, 1),
    "U8": (torch.uint8, 1), "BOOL": (torch.bool, 1), "F8_E4M3": (torch.float8_e4m3fn, 1),
    "F8_E5M2": (torch.float8_e5m2, 1), "U16": (torch.uint16, 2), "U32": (torch.uint32, 4), "U64": (torch.uint64, 8),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}


class SafeTensorsError(ValueError):
    pass


class SafeTensorsFile:
    def __init__(self, path):
        self.path = Path(path)
        self._f = open(self.path, "rb")
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        if len(self._mm) < 8:
            raise SafeTensorsError(f"{path}: truncated")
        (n,) = struct.unpack_from("<Q", self._mm, 0)
        if 8 + n > len(self._mm) or n > 100 * 1024 * 1024:
            raise SafeTensorsError(f"{path}: bad header length {n}")
        header = json.loads(bytes(self._mm[8:8 + n]).decode("utf-8"))
        self.metadata: Dict[str, str] = header.pop("__metadata__", {}) or {}
        self.entries: Dict[str, Dict[str, Any]] = header
        self.data_start = 8 + n
        for name, e in header.items():
            if e["dtype"] not in _DTYPES:
                raise SafeTensorsError(f"{name}: unsupported dtype {e['dtype']}")
            a, b = e["data_offsets"]
            numel = int(np.prod(e["shape"])) if e["shape"] else 1
            if b - a != numel * _DTYPES[e["dtype"]][1] or self.data_start + b > len(self._mm):
                raise SafeTensorsError(f"{name}: data range does not match shape/dtype")

    def keys(self) -> Iterable[str]:
        return self.entries.keys()

    def meta(self, name: str):
        e = self.entries[name]
        return _DTYPES[e["dtype"]][0], tuple(e["shape"])

    def tensor(self, name: str) -> torch.Tensor:
        """Zero-copy view into the mapping (read-only memory: clone before writing)."""
        e = self.entries[name]
        dt, _ = _DTYPES[e["dtype"]]
        a, b = e["data_offsets"]
        if b == a:
            return torch.empty(tuple(e["shape"]), dtype=dt)
        raw = torch.frombuffer(self._mm, dtype=torch.uint8, count=b - a, offset=self.data_start + a)
        return raw.view(dt).reshape(tuple(e["shape"]))

    def close(self):
        try:
            self._mm.close()
        except BufferError:
            pass  # live tensor views keep the mapping alive
        self._f.close()


class SafeTensorsModel:
    """A directory (or single file) of SafeTensors shards presented as one name -> tensor mapping."""

    def __init__(self, path):
        p = Path(path)
        self.files: List[SafeTensorsFile] = []
        self.where: Dict[str, SafeTensorsFile] = {}
        if p.is_file():
            shards = [p]
        else:
            index = p / "model.safetensors.index.json"
            if index.exists():
                wm = json.loads(index.read_text())["weight_map"]
                shards = sorted({p / v for v in wm.values()})
            else:
                shards = sorted(p.glob("*.safetensors"))
        if not shards:
            raise SafeTensorsError(f"no .safetensors files under {path}")
        for s in shards:
            f = SafeTensorsFile(s)
            self.files.append(f)
            for k in f.keys():
                self.where[k] = f
        self.metadata: Dict[str, str] = {}
        for f in self.files:
            self.metadata.update(f.metadata)

    def keys(self):
        return self.where.keys()

    def __contains__(self, k):
        return k in self.where

    def meta(self, name):
        return self.where[name].meta(name)

    def tensor(self, name) -> torch.Tensor:
        return self.where[name].tensor(name)

    def gllm_config(self) -> Optional[dict]:
        raw = self.metadata.get("gllm_config")
        return json.loads(raw) if raw else None


def save_file(tensors: Dict[str, torch.Tensor], path, metadata: Optional[Dict[str, str]] = None):
    header: Dict[str, Any] = {}
    if metadata:
        header["__metadata__"] = {k: str(v) for k, v in metadata.items()}
    off = 0
    blobs = []
    for name, t in tensors.items():
        t = t.detach().cpu().contiguous()
        if t.dtype not in _NAMES:
            raise SafeTensorsError(f"{name}: dtype {t.dtype} cannot be stored")
        raw = t.reshape(-1).view(torch.uint8).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + len(raw)]}
        off += len(raw)
        blobs.append(raw)
    hj = json.dumps(header, separators=(",", ":")).encode("utf-8")
    hj += b" " * ((-len(hj)) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for b in blobs:
            f.write(b)
