"""GGUF v2/v3 container: memory-mapped reader, metadata accessors, tensor views, and a writer (tests,
converters).

Reference parity: ``loader/gguf/reader.rs:26-570`` (magic 0x46554747, version, ``general.alignment`` default
32, dimensions stored innermost-first, tensor offsets relative to the aligned data section, tokenizer arrays
``tokenizer.ggml.*``, multi-file models), ``types.rs`` (dtype table) and ``slice.rs`` (zero-copy slices).
"""
from __future__ import annotations

import mmap
import struct
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Dict, List, Optional

import numpy as np
import torch

from . import quant

GGUF_MAGIC = 0x46554747
(T_U8, T_I8, T_U16, T_I16, T_U32, T_I32, T_F32, T_BOOL, T_STR, T_ARR, T_U64, T_I64, T_F64) = range(13)
_SCALAR = {T_U8: "<B", T_I8: "<b", T_U16: "<H", T_I16: "<h", T_U32: "<I", T_I32: "<i", T_F32: "<f", T_BOOL: "<?",
           T_U64: "<Q", T_I64: "<q", T_F64: "<d"}
_NP = {T_U8: np.uint8, T_I8: np.int8, T_U16: np.uint16, T_I16: np.int16, T_U32: np.uint32, T_I32: np.int32,
       T_F32: np.float32, T_BOOL: np.bool_, T_U64: np.uint64, T_I64: np.int64, T_F64: np.float64}


class GgufError(ValueError):
    pass


@dataclass
class GgufTensorInfo:
    name: str
    shape: tuple  # outermost-first (PyTorch order); the file stores innermost-first
    type_id: int
    offset: int   # relative to the data section
    n_elems: int
    n_bytes: int

    @property
    def type_name(self) -> str:
        return quant.TYPES[self.type_id].name


class _Cursor:
    def __init__(self, buf, pos=0):
        self.buf, self.pos = buf, pos

    def read(self, fmt):
        v = struct.unpack_from(fmt, self.buf, self.pos)[0]
        self.pos += struct.calcsize(fmt)
        return v

    def string(self, version):
        n = self.read("<Q") if version >= 2 else self.read("<I")
        if self.pos + n > len(self.buf):
            raise GgufError("string runs past the end of the file")
        s = bytes(self.buf[self.pos:self.pos + n]).decode("utf-8", "replace")
        self.pos += n
        return s

    def value(self, t, version):
        if t in _SCALAR:
            return self.read(_SCALAR[t])
        if t == T_STR:
            return self.string(version)
        if t == T_ARR:
            et = self.read("<I")
            n = self.read("<Q") if version >= 2 else self.read("<I")
            if et in _NP:
                dt = np.dtype(_NP[et]).newbyteorder("<")
                arr = np.frombuffer(self.buf, dtype=dt, count=n, offset=self.pos)
                self.pos += n * dt.itemsize
                return arr
            return [self.value(et, version) for _ in range(n)]
        raise GgufError(f"unknown metadata value type {t}")


class GgufFile:
    """One ``.gguf`` file, memory mapped. Tensor payloads are never copied until dequantised."""

    def __init__(self, path):
        self.path = Path(path)
        self._f = open(self.path, "rb")
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        buf = memoryview(self._mm)
        c = _Cursor(buf)
        if c.read("<I") != GGUF_MAGIC:
            raise GgufError(f"{path}: not a GGUF file")
        self.version = c.read("<I")
        if self.version not in (1, 2, 3):
            raise GgufError(f"{path}: unsupported GGUF version {self.version}")
        n_tensors = c.read("<Q") if self.version >= 2 else c.read("<I")
        n_kv = c.read("<Q") if self.version >= 2 else c.read("<I")
        self.metadata: Dict[str, Any] = {}
        for _ in range(n_kv):
            key = c.string(self.version)
            t = c.read("<I")
            self.metadata[key] = c.value(t, self.version)
        self.alignment = int(self.metadata.get("general.alignment", 32))
        self.tensors: Dict[str, GgufTensorInfo] = {}
        for _ in range(n_tensors):
            name = c.string(self.version)
            nd = c.read("<I")
            dims = [c.read("<Q") if self.version >= 2 else c.read("<I") for _ in range(nd)]
            type_id = c.read("<I")
            off = c.read("<Q")
            if type_id not in quant.TYPES:
                raise GgufError(f"tensor {name}: unknown ggml type {type_id}")
            n = int(np.prod(dims)) if dims else 1
            qt = quant.TYPES[type_id]
            if dims and dims[0] % qt.block_elems:
                raise GgufError(f"tensor {name}: row length {dims[0]} is not a multiple of the {qt.name} block")
            self.tensors[name] = GgufTensorInfo(name, tuple(reversed(dims)), type_id, off, n, quant.nbytes(type_id, n))
        self.data_start = (c.pos + self.alignment - 1) // self.alignment * self.alignment
        for ti in self.tensors.values():
            if self.data_start + ti.offset + ti.n_bytes > len(buf):
                raise GgufError(f"tensor {ti.name} runs past the end of the file")
        self._buf = buf

    # ------------------------------------------------------------------------------------------
    def raw(self, name: str) -> memoryview:
        ti = self.tensors[name]
        s = self.data_start + ti.offset
        return self._buf[s:s + ti.n_bytes]

    def tensor(self, name: str, dtype=torch.float32) -> torch.Tensor:
        """Dequantised tensor in PyTorch shape order."""
        ti = self.tensors[name]
        t = quant.dequantize(ti.type_id, self.raw(name), ti.n_elems).reshape(ti.shape)
        return t if dtype == torch.float32 else t.to(dtype)

    def architecture(self) -> str:
        return str(self.metadata.get("general.architecture", "llama"))

    def get(self, key: str, default=None):
        return self.metadata.get(key, default)

    def arch_get(self, key: str, default=None):
        return self.metadata.get(f"{self.architecture()}.{key}", default)

    def tokenizer_tokens(self) -> Optional[List[str]]:
        return self.metadata.get("tokenizer.ggml.tokens")

    def tokenizer_merges(self) -> Optional[List[str]]:
        return self.metadata.get("tokenizer.ggml.merges")

    def file_type_summary(self) -> Dict[str, int]:
        out: Dict[str, int] = {}
        for ti in self.tensors.values():
            out[ti.type_name] = out.get(ti.type_name, 0) + 1
        return out

    def close(self):
        self._buf = None
        try:
            self._mm.close()
        except BufferError:
            pass
        self._f.close()


def open_multi(paths) -> List[GgufFile]:
    """Split models (``-00001-of-0000N.gguf``): open every shard; tensors are disjoint across shards."""
    return [GgufFile(p) for p in sorted(map(str, paths))]


# ------------------------------------------------------------------------------------------------
# writer
# ------------------------------------------------------------------------------------------------
def _w_string(out: bytearray, s: str):
    b = s.encode("utf-8")
    out += struct.pack("<Q", len(b)) + b


def _w_value(out: bytearray, v):
    if isinstance(v, bool):
        out += struct.pack("<I?", T_BOOL, v)
    elif isinstance(v, int):
        out += struct.pack("<I", T_U32 if 0 <= v < 2 ** 32 else T_I64)
        out += struct.pack("<I" if 0 <= v < 2 ** 32 else "<q", v)
    elif isinstance(v, float):
        out += struct.pack("<If", T_F32, v)
    elif isinstance(v, str):
        out += struct.pack("<I", T_STR)
        _w_string(out, v)
    elif isinstance(v, (list, tuple, np.ndarray)):
        out += struct.pack("<I", T_ARR)
        seq = list(v)
        if seq and isinstance(seq[0], str):
            out += struct.pack("<IQ", T_STR, len(seq))
            for s in seq:
                _w_string(out, s)
        elif seq and isinstance(seq[0], float):
            out += struct.pack("<IQ", T_F32, len(seq)) + np.asarray(seq, "<f4").tobytes()
        else:
            out += struct.pack("<IQ", T_I32, len(seq)) + np.asarray(seq, "<i4").tobytes()
    else:
        raise TypeError(f"cannot store metadata value of type {type(v)}")


def write_gguf(path, metadata: Dict[str, Any], tensors: Dict[str, Any], alignment: int = 32):
    """tensors: name -> torch tensor (stored F32/F16/BF16) or (type_name, shape, raw_bytes) for quantised data."""
    head = bytearray(struct.pack("<IIQQ", GGUF_MAGIC, 3, len(tensors), len(metadata)))
    for k, v in metadata.items():
        _w_string(head, k)
        _w_value(head, v)
    blobs, off = [], 0
    for name, t in tensors.items():
        if isinstance(t, tuple):
            tname, shape, raw = t
            tid = quant.BY_NAME[tname].id
        else:
            tt = t.detach().cpu().contiguous()
            tid = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 30}[tt.dtype]
            shape = tuple(tt.shape)
            raw = tt.view(torch.uint8).numpy().tobytes() if tt.dtype != torch.bfloat16 else tt.view(torch.int16).numpy().tobytes()
        _w_string(head, name)
        dims = list(reversed(shape))
        head += struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims)
        head += struct.pack("<IQ", tid, off)
        pad = (-len(raw)) % alignment
        blobs.append(raw + b"\0" * pad)
        off += len(raw) + pad
    pad = (-len(head)) % alignment
    with open(path, "wb") as f:
        f.write(head + b"\0" * pad)
        for b in blobs:
            f.write(b)
