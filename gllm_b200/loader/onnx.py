"""ONNX checkpoints: a dependency-free protobuf wire reader that extracts the graph's initializers (weights,
including external-data tensors) and the node list, enough to load encoder / reranker exports.

Reference parity: ``loader/onnx/*`` (protobuf parse, initializers, external data, pattern matching to fused
ops). Only the fields the loader needs are decoded: ModelProto.graph(7) -> GraphProto.node(1) /
initializer(5) -> TensorProto{dims(1), data_type(2), float_data(4), int64_data(7), name(8), raw_data(9),
external_data(13), data_location(14)}; NodeProto{input(1), output(2), name(3), op_type(4)}.
"""
from __future__ import annotations

import struct
from pathlib import Path
from typing import Dict, List, Tuple

import numpy as np
import torch

from .loader import TensorProvider
from .name_map import match_tensor_role

_ONNX_DTYPES = {1: np.float32, 2: np.uint8, 3: np.int8, 5: np.int16, 6: np.int32, 7: np.int64, 9: np.bool_,
                10: np.float16, 11: np.float64, 12: np.uint32, 13: np.uint64}


def _varint(buf, pos):
    out = shift = 0
    while True:
        b = buf[pos]
        pos += 1
        out |= (b & 0x7F) << shift
        if not b & 0x80:
            return out, pos
        shift += 7


def _fields(buf):
    """Yield (field number, wire type, value) over one message; length-delimited values are memoryviews."""
    pos, n = 0, len(buf)
    while pos < n:
        key, pos = _varint(buf, pos)
        fn, wt = key >> 3, key & 7
        if wt == 0:
            v, pos = _varint(buf, pos)
        elif wt == 1:
            v = bytes(buf[pos:pos + 8]); pos += 8
        elif wt == 2:
            ln, pos = _varint(buf, pos)
            v = buf[pos:pos + ln]; pos += ln
        elif wt == 5:
            v = bytes(buf[pos:pos + 4]); pos += 4
        else:
            raise ValueError(f"unsupported protobuf wire type {wt}")
        yield fn, wt, v


def _parse_tensor(buf, base_dir: Path):
    dims: List[int] = []
    dtype = 1
    name = ""
    raw = None
    floats: List[float] = []
    int64s: List[int] = []
    external: Dict[str, str] = {}
    for fn, wt, v in _fields(buf):
        if fn == 1:
            if wt == 0:
                dims.append(v)
            else:  # packed
                p = 0
                while p < len(v):
                    d, p = _varint(v, p)
                    dims.append(d)
        elif fn == 2:
            dtype = v
        elif fn == 4:
            floats += list(np.frombuffer(bytes(v), "<f4")) if wt == 2 else [struct.unpack("<f", v)[0]]
        elif fn == 7:
            if wt == 2:
                p = 0
                while p < len(v):
                    d, p = _varint(v, p)
                    int64s.append(d)
            else:
                int64s.append(v)
        elif fn == 8:
            name = bytes(v).decode("utf-8")
        elif fn == 9:
            raw = bytes(v)
        elif fn == 13:
            kv = {f: bytes(x).decode() for f, _, x in _fields(v) if f in (1, 2)}
            external[kv.get(1, "")] = kv.get(2, "")
    np_dt = _ONNX_DTYPES.get(dtype)
    count = int(np.prod(dims)) if dims else 1
    if external:
        p = base_dir / external["location"]
        off, ln = int(external.get("offset", 0)), int(external.get("length", 0)) or None
        with open(p, "rb") as f:
            f.seek(off)
            raw = f.read(ln) if ln else f.read()
    if dtype == 16:  # bfloat16
        arr = torch.frombuffer(bytearray(raw), dtype=torch.bfloat16, count=count).reshape(dims)
        return name, arr
    if np_dt is None:
        return name, None
    if raw is not None:
        arr = np.frombuffer(raw, dtype=np.dtype(np_dt).newbyteorder("<"), count=count)
    elif floats:
        arr = np.asarray(floats, np.float32)
    else:
        arr = np.asarray(int64s, np.int64).astype(np_dt)
    return name, torch.from_numpy(arr.reshape(dims).copy())


def read_onnx(path) -> Tuple[Dict[str, torch.Tensor], List[dict]]:
    path = Path(path)
    buf = memoryview(path.read_bytes())
    tensors: Dict[str, torch.Tensor] = {}
    nodes: List[dict] = []
    for fn, wt, v in _fields(buf):
        if fn != 7 or wt != 2:
            continue
        for gfn, gwt, gv in _fields(v):
            if gfn == 5 and gwt == 2:
                name, t = _parse_tensor(gv, path.parent)
                if t is not None:
                    tensors[name] = t
            elif gfn == 1 and gwt == 2:
                node = {"input": [], "output": [], "name": "", "op_type": ""}
                for nfn, nwt, nv in _fields(gv):
                    if nfn == 1:
                        node["input"].append(bytes(nv).decode())
                    elif nfn == 2:
                        node["output"].append(bytes(nv).decode())
                    elif nfn == 3:
                        node["name"] = bytes(nv).decode()
                    elif nfn == 4:
                        node["op_type"] = bytes(nv).decode()
                nodes.append(node)
    return tensors, nodes


def fused_patterns(nodes: List[dict]) -> Dict[str, int]:
    """Count the op patterns the engine fuses (MatMul+Add -> linear, Erf chain -> GELU, LayerNormalization)."""
    ops = [n["op_type"] for n in nodes]
    out = {"linear": 0, "gelu": ops.count("Erf") + ops.count("Gelu"),
           "layernorm": ops.count("LayerNormalization") + ops.count("ReduceMean") // 2, "softmax": ops.count("Softmax")}
    produced = {o: n for n in nodes for o in n["output"]}
    for n in nodes:
        if n["op_type"] == "Add" and any(produced.get(i, {}).get("op_type") == "MatMul" for i in n["input"]):
            out["linear"] += 1
    return out


class OnnxProvider(TensorProvider):
    def __init__(self, path, dtype=torch.bfloat16):
        super().__init__()
        self.dtype = dtype
        self.tensors, self.nodes = read_onnx(path)
        # MatMul weights in ONNX exports are stored [in, out]: remember which initializers feed a MatMul
        self._transposed = {n["input"][1] for n in self.nodes if n["op_type"] == "MatMul" and len(n["input"]) > 1}
        for n, t in self.tensors.items():
            self.shapes[n] = tuple(t.shape)
            canon = match_tensor_role(n)[2]
            if canon:
                self.canon_to_external[canon] = n

    def get(self, name):
        ext = self.canon_to_external[name]
        t = self.tensors[ext]
        if ext in self._transposed and t.dim() == 2:
            t = t.t().contiguous()
        if name.rsplit(".", 1)[-1].endswith("norm"):
            return t.float()
        return t.to(self.dtype) if t.is_floating_point() else t
