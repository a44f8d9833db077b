"""The native ``.gllm`` container: one file holding metadata, a tensor table and payloads laid out for mmap.

Reference parity: ``loader/gllm/*`` — 64-byte header, 72-byte tensor entries, string table, MessagePack
metadata, native-quant payloads, converters from GGUF / SafeTensors. Layout here (little endian):

    header   64 B   magic "GLLMB200", u32 version, u32 n_tensors, u64 entries_off, u64 strings_off,
                    u64 strings_len, u64 meta_off, u64 meta_len, u64 data_off
    entry    72 B   u64 name_off, u32 name_len, u32 dtype (quant type id, or 100+ for torch dtypes), u32 ndim,
                    u32 reserved, u64 shape[4], u64 data_off (relative to data section), u64 nbytes
    strings         concatenated UTF-8 names
    metadata        MessagePack map (config, tokenizer file names, source format, quantisation summary)
    data            256-byte aligned payloads
"""
from __future__ import annotations

import mmap
import struct
from pathlib import Path
from typing import Dict

import msgpack
import numpy as np
import torch

from . import quant
from .loader import TensorProvider
from .name_map import match_tensor_role

MAGIC = b"GLLMB200"
HEADER = struct.Struct("<8sIIQQQQQQ")
ENTRY = struct.Struct("<QIIII4QQQ")
_TORCH_IDS = {torch.float32: 100, torch.float16: 101, torch.bfloat16: 102, torch.float8_e4m3fn: 103,
              torch.float8_e5m2: 104, torch.uint8: 105, torch.int8: 106, torch.int32: 107, torch.int64: 108}
_TORCH_BY_ID = {v: k for k, v in _TORCH_IDS.items()}


def write_gllm(path, tensors: Dict[str, object], metadata: dict):
    """tensors: name -> torch tensor, or (quant type name, shape, raw bytes) for block-quantised payloads."""
    names = b""
    entries = []
    blobs = []
    off = 0
    for name, t in tensors.items():
        nb = name.encode("utf-8")
        if isinstance(t, tuple):
            tname, shape, raw = t
            dtype_id = quant.BY_NAME[tname].id
        else:
            tt = t.detach().cpu().contiguous()
            dtype_id = _TORCH_IDS[tt.dtype]
            shape = tuple(tt.shape)
            raw = tt.reshape(-1).view(torch.uint8).numpy().tobytes()
        if len(shape) > 4:
            raise ValueError(f"{name}: more than 4 dimensions")
        sh = list(shape) + [0] * (4 - len(shape))
        entries.append((len(names), len(nb), dtype_id, len(shape), 0, *sh, off, len(raw)))
        names += nb
        pad = (-len(raw)) % 256
        blobs.append(raw + b"\0" * pad)
        off += len(raw) + pad
    meta = msgpack.packb(metadata, use_bin_type=True)
    entries_off = HEADER.size
    strings_off = entries_off + ENTRY.size * len(entries)
    meta_off = strings_off + len(names)
    data_off = (meta_off + len(meta) + 255) // 256 * 256
    with open(path, "wb") as f:
        f.write(HEADER.pack(MAGIC, 1, len(entries), entries_off, strings_off, len(names), meta_off, len(meta), data_off))
        for e in entries:
            f.write(ENTRY.pack(*e))
        f.write(names)
        f.write(meta)
        f.write(b"\0" * (data_off - meta_off - len(meta)))
        for b in blobs:
            f.write(b)


class GllmFile:
    def __init__(self, path):
        self.path = Path(path)
        self._f = open(self.path, "rb")
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        magic, ver, n, eoff, soff, slen, moff, mlen, doff = HEADER.unpack_from(self._mm, 0)
        if magic != MAGIC:
            raise ValueError(f"{path}: not a .gllm file")
        self.version, self.data_off = ver, doff
        self.metadata = msgpack.unpackb(bytes(self._mm[moff:moff + mlen]), raw=False) if mlen else {}
        self.entries: Dict[str, tuple] = {}
        for i in range(n):
            e = ENTRY.unpack_from(self._mm, eoff + i * ENTRY.size)
            name = bytes(self._mm[soff + e[0]:soff + e[0] + e[1]]).decode("utf-8")
            shape = tuple(int(x) for x in e[5:5 + e[3]])
            self.entries[name] = (e[2], shape, e[9], e[10])

    def tensor(self, name: str) -> torch.Tensor:
        dtype_id, shape, off, nbytes = self.entries[name]
        start = self.data_off + off
        if dtype_id >= 100:
            dt = _TORCH_BY_ID[dtype_id]
            if nbytes == 0:
                return torch.empty(shape, dtype=dt)
            return torch.frombuffer(self._mm, dtype=torch.uint8, count=nbytes, offset=start).view(dt).reshape(shape)
        n = int(np.prod(shape))
        return quant.dequantize(dtype_id, memoryview(self._mm)[start:start + nbytes], n).reshape(shape)


class GllmProvider(TensorProvider):
    def __init__(self, path, dtype=torch.bfloat16):
        super().__init__()
        self.file = GllmFile(path)
        self.metadata = self.file.metadata
        self.dtype = dtype
        for n, (dtype_id, shape, _, _) in self.file.entries.items():
            self.shapes[n] = shape
            canon = n if (n.startswith("L") or n in ("embed_tokens", "final_norm", "lm_head")) else match_tensor_role(n)[2]
            if canon:
                self.canon_to_external[canon] = n
            if dtype_id < 100 and dtype_id not in (0, 1, 30):
                qn = quant.TYPES[dtype_id].name
                self.quant_summary[qn] = self.quant_summary.get(qn, 0) + 1

    def get(self, name: str) -> torch.Tensor:
        t = self.file.tensor(self.canon_to_external[name])
        if name.rsplit(".", 1)[-1].endswith("norm"):
            return t.float()
        return t.to(self.dtype) if t.is_floating_point() else t


def convert_to_gllm(loaded, out_path, quantize: str = ""):
    """SafeTensors / GGUF model -> .gllm with canonical names. ``quantize``: "", "Q8_0", "Q4_K", ... for 2-D weights."""
    tensors = {}
    for name in loaded.weights.names():
        if "stacked" in name:
            continue
        t = loaded.weights.get(name)
        base = name.rsplit(".", 1)[-1]
        if quantize and t.dim() == 2 and not base.endswith("norm") and t.shape[1] % quant.BY_NAME[quantize].block_elems == 0 \
                and base not in ("embed_tokens",):
            raw = quant.QUANTIZERS[quantize](t.float().numpy())
            tensors[name] = (quantize, tuple(t.shape), raw)
        else:
            tensors[name] = t
    meta = {"config": {k: v for k, v in loaded.config.to_dict().items() if isinstance(v, (int, float, str, bool, list))},
            "source_format": loaded.format.value, "quantize": quantize}
    write_gllm(out_path, tensors, meta)
    return out_path
