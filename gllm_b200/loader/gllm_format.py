"""The native ``.gllm`` container: one file holding metadata, a tensor table and payloads laid out for mmap.

Two layouts are read, chosen by the magic; the first one is written.

**Reference layout** (src/loader/gllm/types.rs:75-200, reader.rs:58-140, writer.rs:59-75; little endian):

    header   64 B   u32 magic 0x4D4C4C47 ("GLLM") @0, u32 version (1) @4, u32 flags (bit 0: some tensor is quantised)
                    @8, u64 meta_offset @12, u32 tensor_count @20, u64 tensor_dir_offset @24, u64 data_offset @32,
                    u32 page_size @40, zero padding to 64
    entry    72 B   u32 name_offset, u16 name_len, u8 ndim, u8 dtype, u64 shape[4] @8, u8 quant_format @40,
                    u16 quant_block_size @41, u8 scale_dtype @43, u8 zp_type @44, 3 B padding, u64 data_offset @48
                    (relative to the data region), u64 compressed_size @56, u64 original_size @64
    strings         UTF-8 names, directly after the tensor directory
    metadata        MessagePack map at meta_offset (up to data_offset)
    data            page-aligned region; a quantised tensor occupies compressed_size bytes, a plain one original_size

    dtype bytes: 0 F32, 1 F16, 2 BF16, 3 U8, 4 I8, 5 I32, 6 I64.  quant_format bytes: 0 none, 10-15 Q4_0..Q8_1,
    20-25 Q2_K..Q8_K, 30-38 IQ1_S..IQ4_XS, 40 AWQ4, 41 GPTQ4, 42 Squeeze, 50 / 51 fp8 e4m3 / e5m2, 52 MXFP4, 53 NVFP4.

Every offset is checked against the file size before it is used (tensor directory, names, metadata, payloads), and
duplicate names are rejected, as the reference's reader does.

**Private layout** (magic "GLLMB200", written by earlier versions of this package): 64-byte header with explicit
string / metadata lengths and 72-byte entries with u32 fields; still readable, no longer written.
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

GLLM_MAGIC = 0x4D4C4C47
GLLM_VERSION = 1
HEADER_SIZE = 64
REF_HEADER = struct.Struct("<IIIQIQQI")                 # 44 bytes used, zero padded to 64
REF_ENTRY = struct.Struct("<IHBB4QBHBB3xQQQ")           # 72 bytes
assert REF_HEADER.size == 44 and REF_ENTRY.size == 72
_DTYPE_CODE = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2, torch.uint8: 3, torch.int8: 4, torch.int32: 5,
               torch.int64: 6}
_DTYPE_BY_CODE = {v: k for k, v in _DTYPE_CODE.items()}
_QUANT_CODE = {"Q4_0": 10, "Q4_1": 11, "Q5_0": 12, "Q5_1": 13, "Q8_0": 14, "Q8_1": 15, "Q2_K": 20, "Q3_K": 21, "Q4_K": 22,
               "Q5_K": 23, "Q6_K": 24, "Q8_K": 25, "IQ1_S": 30, "IQ1_M": 31, "IQ2_XXS": 32, "IQ2_XS": 33, "IQ2_S": 34,
               "IQ3_XXS": 35, "IQ3_S": 36, "IQ4_NL": 37, "IQ4_XS": 38, "AWQ4": 40, "GPTQ4": 41, "SQUEEZE": 42,
               "FP8_E4M3": 50, "FP8_E5M2": 51, "MXFP4": 52, "NVFP4": 53}
_QUANT_BY_CODE = {v: k for k, v in _QUANT_CODE.items()}

PRIVATE_MAGIC = b"GLLMB200"
PRIVATE_HEADER = struct.Struct("<8sIIQQQQQQ")
PRIVATE_ENTRY = struct.Struct("<QIIII4QQQ")
_TORCH_IDS = {torch.float32: 100, torch.float16: 101, torch.bfloat16: 102, torch.float8_e4m3fn: 103,
              torch.float8_e5m2: 104, torch.uint8: 105, torch.int8: 106, torch.int32: 107, torch.int64: 108}
_TORCH_BY_ID = {v: k for k, v in _TORCH_IDS.items()}


class GllmFormatError(ValueError):
    """A ``.gllm`` file that cannot be trusted: bad magic / version, or an offset that leaves the file."""


def write_gllm(path, tensors: Dict[str, object], metadata: dict, page_size: int = 4096):
    """Write the reference layout. tensors: name -> torch tensor, or (quant type name, shape, raw bytes) for
    block-quantised payloads (GGML block formats; fp8 tensors are stored as quant_format 50 / 51 over U8)."""
    names = b""
    entries, blobs = [], []
    off, any_quant = 0, False
    for name, t in tensors.items():
        nb = name.encode("utf-8")
        qfmt, qblock = 0, 0
        if isinstance(t, tuple):
            tname, shape, raw = t
            if tname not in _QUANT_CODE:
                raise ValueError(f"{name}: no .gllm quant_format code for {tname}")
            qfmt, qblock, dcode = _QUANT_CODE[tname], int(quant.BY_NAME[tname].block_elems), 3
            original = int(np.prod(shape)) * 4
            any_quant = True
        else:
            tt = t.detach().cpu().contiguous()
            shape = tuple(tt.shape)
            if tt.dtype in (torch.float8_e4m3fn, torch.float8_e5m2):
                qfmt, dcode = (50 if tt.dtype == torch.float8_e4m3fn else 51), 3
                original, any_quant = tt.numel() * 4, True
            else:
                dcode = _DTYPE_CODE[tt.dtype]
                original = tt.numel() * tt.element_size()
            raw = tt.reshape(-1).view(torch.uint8).numpy().tobytes()
        if len(shape) > 4:
            raise ValueError(f"{name}: more than 4 dimensions")
        if len(nb) > 0xFFFF:
            raise ValueError(f"{name}: name longer than 65535 bytes")
        sh = list(shape) + [0] * (4 - len(shape))
        entries.append((len(names), len(nb), len(shape), dcode, *sh, qfmt, qblock, 0, 0, off,
                        len(raw) if qfmt else 0, original))
        names += nb
        pad = (-len(raw)) % 256
        blobs.append(raw + b"\0" * pad)
        off += len(raw) + pad
    meta = msgpack.packb(metadata, use_bin_type=True)
    dir_off = HEADER_SIZE
    strings_off = dir_off + REF_ENTRY.size * len(entries)
    meta_off = strings_off + len(names)
    data_off = (meta_off + len(meta) + page_size - 1) // page_size * page_size
    with open(path, "wb") as f:
        f.write(REF_HEADER.pack(GLLM_MAGIC, GLLM_VERSION, 1 if any_quant else 0, meta_off, len(entries), dir_off, data_off,
                                page_size).ljust(HEADER_SIZE, b"\0"))
        for e in entries:
            f.write(REF_ENTRY.pack(*e))
        f.write(names)
        f.write(meta)
        f.write(b"\0" * (data_off - meta_off - len(meta)))
        for b in blobs:
            f.write(b)


class GllmFile:
    """Memory-mapped reader. ``entries[name] = (kind, shape, absolute offset, nbytes)`` where kind is a torch dtype or a
    quant type name."""

    def __init__(self, path):
        self.path = Path(path)
        self._f = open(self.path, "rb")
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        size = len(self._mm)
        if size < HEADER_SIZE:
            raise GllmFormatError(f"{path}: file too small for a header: {size} bytes (need {HEADER_SIZE})")
        self.entries: Dict[str, tuple] = {}
        if bytes(self._mm[:8]) == PRIVATE_MAGIC:
            self._parse_private(size)
        elif struct.unpack_from("<I", self._mm, 0)[0] == GLLM_MAGIC:
            self._parse_reference(size)
        else:
            raise GllmFormatError(f"{path}: not a .gllm file (magic {bytes(self._mm[:4])!r})")

    # ---- reference layout --------------------------------------------------------------------------------
    def _parse_reference(self, size: int):
        _, ver, flags, meta_off, count, dir_off, data_off, page = REF_HEADER.unpack_from(self._mm, 0)
        if ver != GLLM_VERSION:
            raise GllmFormatError(f"{self.path}: unsupported version {ver} (expected {GLLM_VERSION})")
        self.version, self.flags, self.page_size, self.layout = ver, flags, page, "reference"
        dir_end = dir_off + count * REF_ENTRY.size
        if dir_end > size:
            raise GllmFormatError(f"{self.path}: tensor directory [{dir_off}..{dir_end}) exceeds file size {size}")
        if meta_off > size or data_off > size or meta_off > data_off:
            raise GllmFormatError(f"{self.path}: metadata offset {meta_off} / data offset {data_off} exceed file size {size}")
        for i in range(count):
            (noff, nlen, ndim, dcode, s0, s1, s2, s3, qfmt, qblock, _sdt, _zp, rel, csize, osize) = \
                REF_ENTRY.unpack_from(self._mm, dir_off + i * REF_ENTRY.size)
            n0 = dir_end + noff
            if n0 + nlen > data_off:
                raise GllmFormatError(f"{self.path}: string table [{n0}..{n0 + nlen}) exceeds file size {size}")
            name = bytes(self._mm[n0:n0 + nlen]).decode("utf-8")
            if ndim > 4:
                raise GllmFormatError(f"{self.path}: tensor {name!r} has {ndim} dimensions")
            nbytes = csize if qfmt else osize
            start = data_off + rel
            if start + nbytes > size:
                raise GllmFormatError(f"{self.path}: tensor {name!r} [{start}..{start + nbytes}) exceeds file size {size}")
            if name in self.entries:
                raise GllmFormatError(f"{self.path}: duplicate tensor name {name!r}")
            shape = tuple(int(x) for x in (s0, s1, s2, s3)[:ndim])
            if qfmt == 0 or qfmt in (1, 2, 3):
                if qfmt:        # a "quantised" entry that is plain bf16 / f16 / f32
                    kind = {1: torch.bfloat16, 2: torch.float16, 3: torch.float32}[qfmt]
                elif dcode in _DTYPE_BY_CODE:
                    kind = _DTYPE_BY_CODE[dcode]
                else:
                    raise GllmFormatError(f"{self.path}: tensor {name!r}: invalid dtype {dcode}")
            elif qfmt == 50:
                kind = torch.float8_e4m3fn
            elif qfmt == 51:
                kind = torch.float8_e5m2
            elif qfmt in _QUANT_BY_CODE:
                kind = _QUANT_BY_CODE[qfmt]
            else:
                raise GllmFormatError(f"{self.path}: tensor {name!r}: invalid quant_format {qfmt}")
            self.entries[name] = (kind, shape, start, int(nbytes))
        raw_meta = bytes(self._mm[meta_off:data_off]) if data_off > meta_off else b""
        self.metadata = {}
        if raw_meta.strip(b"\0"):
            up = msgpack.Unpacker(raw=False)
            up.feed(raw_meta)
            self.metadata = next(iter(up))
            if not isinstance(self.metadata, dict):
                raise GllmFormatError(f"{self.path}: metadata is not a map")

    # ---- private layout (read only) ---------------------------------------------------------------------
    def _parse_private(self, size: int):
        _, ver, n, eoff, soff, slen, moff, mlen, doff = PRIVATE_HEADER.unpack_from(self._mm, 0)
        self.version, self.flags, self.page_size, self.layout = ver, 0, 256, "private"
        if eoff + n * PRIVATE_ENTRY.size > size or soff + slen > size or moff + mlen > size or doff > size:
            raise GllmFormatError(f"{self.path}: a section of the private layout leaves the file ({size} bytes)")
        self.metadata = msgpack.unpackb(bytes(self._mm[moff:moff + mlen]), raw=False) if mlen else {}
        for i in range(n):
            e = PRIVATE_ENTRY.unpack_from(self._mm, eoff + i * PRIVATE_ENTRY.size)
            if e[0] + e[1] > slen or doff + e[9] + e[10] > size or e[3] > 4:
                raise GllmFormatError(f"{self.path}: entry {i} of the private layout leaves the file")
            name = bytes(self._mm[soff + e[0]:soff + e[0] + e[1]]).decode("utf-8")
            shape = tuple(int(x) for x in e[5:5 + e[3]])
            kind = _TORCH_BY_ID[e[2]] if e[2] >= 100 else quant.TYPES[e[2]].name
            self.entries[name] = (kind, shape, doff + e[9], e[10])

    def tensor(self, name: str) -> torch.Tensor:
        kind, shape, start, nbytes = self.entries[name]
        if isinstance(kind, torch.dtype):
            if nbytes == 0:
                return torch.empty(shape, dtype=kind)
            return torch.frombuffer(self._mm, dtype=torch.uint8, count=nbytes, offset=start).view(kind).reshape(shape)
        n = int(np.prod(shape))
        return quant.dequantize(quant.BY_NAME[kind].id, memoryview(self._mm)[start:start + nbytes], n).reshape(shape)


class GllmProvider(TensorProvider):
    def __init__(self, path, dtype=torch.bfloat16):
        super().__init__()
        self.file = GllmFile(path)
        self.metadata = self.file.metadata
        self.dtype = dtype
        for n, (kind, shape, _, _) in self.file.entries.items():
            self.shapes[n] = shape
            canon = n if (n.startswith("L") or n in ("embed_tokens", "final_norm", "lm_head")) else match_tensor_role(n)[2]
            if canon:
                self.canon_to_external[canon] = n
            if not isinstance(kind, torch.dtype):
                self.quant_summary[kind] = self.quant_summary.get(kind, 0) + 1

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
