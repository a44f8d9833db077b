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
        # initializers without usable names (``onnx::MatMul_123``): the graph structure names them
        self.fused_ops = OnnxGraph(self.nodes, self.tensors.keys()).fuse()
        for canon, ext in name_encoder_weights(self.fused_ops).items():
            self.canon_to_external.setdefault(canon, ext)

    def get(self, name):
        ext = self.canon_to_external[name]
        t = self.tensors[ext]
        if ext in self._transposed and t.dim() == 2:
            t = t.t().contiguous()
        if name.rsplit(".", 1)[-1].endswith("norm"):
            return t.float()
        return t.to(self.dtype) if t.is_floating_point() else t


# ------------------------------------------------------------------------------------------------
# graph import: pattern matching of the exported operator soup into the ops the engine runs
# ------------------------------------------------------------------------------------------------
class FusedOp:
    """One recovered op: ``kind`` in {embedding, layernorm, linear, gelu, attention, add, other}, the graph values it
    reads / writes and the initializers (weights) it owns."""

    def __init__(self, kind: str, inputs, outputs, weights=None, nodes=None, attrs=None):
        self.kind, self.inputs, self.outputs = kind, list(inputs), list(outputs)
        self.weights, self.nodes, self.attrs = dict(weights or {}), list(nodes or []), dict(attrs or {})

    def __repr__(self):
        return f"FusedOp({self.kind}, in={self.inputs}, out={self.outputs}, w={list(self.weights.values())})"


class OnnxGraph:
    """Producer / consumer view of a node list.

    Reference parity: the reference's ONNX front end matches exported sub-graphs to fused ops before it builds its
    compiler graph (loader/onnx/*: decomposed LayerNorm, erf-GELU, MatMul+Add, the softmax attention core)."""

    def __init__(self, nodes: List[dict], initializers):
        self.nodes = nodes
        self.init = set(initializers)
        self.producer = {o: i for i, n in enumerate(nodes) for o in n["output"]}
        self.consumers: Dict[str, List[int]] = {}
        for i, n in enumerate(nodes):
            for v in n["input"]:
                self.consumers.setdefault(v, []).append(i)

    def prod(self, value):
        i = self.producer.get(value)
        return None if i is None else self.nodes[i]

    def sole_consumer(self, value, op_type=None):
        c = self.consumers.get(value, [])
        if len(c) != 1:
            return None
        n = self.nodes[c[0]]
        return n if (op_type is None or n["op_type"] == op_type) else None

    def _weight_in(self, node):
        return [v for v in node["input"] if v in self.init]

    def _data_in(self, node):
        return [v for v in node["input"] if v not in self.init]

    # ---- patterns ------------------------------------------------------------------------------------
    def match_layernorm(self, start: int):
        """ReduceMean -> Sub -> Pow -> ReduceMean -> Add(eps) -> Sqrt -> Div -> Mul(gamma) -> Add(beta), entered at
        the first ReduceMean; or the native LayerNormalization op."""
        n = self.nodes[start]
        if n["op_type"] == "LayerNormalization":
            w = self._weight_in(n)
            return FusedOp("layernorm", self._data_in(n)[:1], n["output"][:1],
                           {"gamma": w[0] if w else None, "beta": w[1] if len(w) > 1 else None}, [start])
        if n["op_type"] != "ReduceMean":
            return None
        x = n["input"][0]
        sub = next((self.nodes[c] for c in self.consumers.get(n["output"][0], []) if self.nodes[c]["op_type"] == "Sub"), None)
        if sub is None or x not in sub["input"]:
            return None
        chain, cur = [start, self.nodes.index(sub)], sub
        pow_ = next((self.nodes[c] for c in self.consumers.get(sub["output"][0], []) if self.nodes[c]["op_type"] in ("Pow", "Mul")), None)
        if pow_ is None:
            return None
        cur = pow_
        chain.append(self.nodes.index(cur))
        for want in ("ReduceMean", "Add", "Sqrt"):
            cur = self.sole_consumer(cur["output"][0], want)
            if cur is None:
                return None
            chain.append(self.nodes.index(cur))
        div = self.sole_consumer(cur["output"][0], "Div")
        if div is None or sub["output"][0] not in div["input"]:
            return None
        chain.append(self.nodes.index(div))
        out, weights = div["output"][0], {}
        mul = self.sole_consumer(out, "Mul")
        if mul is not None and self._weight_in(mul):
            weights["gamma"], out = self._weight_in(mul)[0], mul["output"][0]
            chain.append(self.nodes.index(mul))
            add = self.sole_consumer(out, "Add")
            if add is not None and self._weight_in(add):
                weights["beta"], out = self._weight_in(add)[0], add["output"][0]
                chain.append(self.nodes.index(add))
        return FusedOp("layernorm", [x], [out], weights, chain)

    def match_gelu(self, start: int):
        """x / sqrt(2) -> Erf -> + 1 -> * x -> * 0.5 (any order of the two multiplies), entered at the Div; or Gelu."""
        n = self.nodes[start]
        if n["op_type"] in ("Gelu", "FastGelu"):
            return FusedOp("gelu", self._data_in(n)[:1], n["output"][:1], nodes=[start])
        if n["op_type"] != "Div":
            return None
        erf = self.sole_consumer(n["output"][0], "Erf")
        if erf is None:
            return None
        x = self._data_in(n)[0]
        add = self.sole_consumer(erf["output"][0], "Add")
        if add is None:
            return None
        chain, cur = [start, self.nodes.index(erf), self.nodes.index(add)], add
        for _ in range(2):
            nxt = self.sole_consumer(cur["output"][0], "Mul")
            if nxt is None:
                break
            cur = nxt
            chain.append(self.nodes.index(cur))
        return FusedOp("gelu", [x], [cur["output"][0]], nodes=chain)

    def match_linear(self, start: int):
        """MatMul(x, W) [-> Add(bias)] or Gemm."""
        n = self.nodes[start]
        if n["op_type"] == "Gemm":
            w = self._weight_in(n)
            return FusedOp("linear", self._data_in(n)[:1], n["output"][:1],
                           {"weight": w[0] if w else None, "bias": w[1] if len(w) > 1 else None}, [start],
                           {"weight_is_in_out": False})
        if n["op_type"] != "MatMul" or len(self._weight_in(n)) != 1:
            return None
        out, weights, chain = n["output"][0], {"weight": self._weight_in(n)[0]}, [start]
        add = self.sole_consumer(out, "Add")
        if add is not None and self._weight_in(add):
            weights["bias"], out = self._weight_in(add)[0], add["output"][0]
            chain.append(self.nodes.index(add))
        return FusedOp("linear", self._data_in(n)[:1], [out], weights, chain, {"weight_is_in_out": True})

    def match_attention(self, start: int):
        """Softmax with a data x data MatMul before it (scores, possibly scaled / masked) and one after it (context)."""
        n = self.nodes[start]
        if n["op_type"] != "Softmax":
            return None
        chain, cur, qk = [start], n, None
        for _ in range(4):                       # walk up through scale (Div / Mul) and mask (Add) to the QK^T MatMul
            p = self.prod(self._data_in(cur)[0]) if self._data_in(cur) else None
            if p is None:
                return None
            chain.append(self.nodes.index(p))
            if p["op_type"] == "MatMul" and not self._weight_in(p):
                qk = p
                break
            if p["op_type"] not in ("Div", "Mul", "Add", "Where", "Cast"):
                return None
            cur = p
        pv = self.sole_consumer(n["output"][0], "MatMul")
        if qk is None or pv is None:
            return None
        chain.append(self.nodes.index(pv))
        v_in = [v for v in pv["input"] if v != n["output"][0]]
        return FusedOp("attention", qk["input"][:2] + v_in[:1], pv["output"][:1], nodes=chain)

    def fuse(self) -> List[FusedOp]:
        """Greedy cover of the node list by the patterns, in graph order; uncovered nodes stay ``other`` ops."""
        used, out = set(), []
        # the attention core is entered at its Softmax, in the middle of the pattern: claim those nodes first
        for i, n in enumerate(self.nodes):
            if n["op_type"] == "Softmax":
                op = self.match_attention(i)
                if op is not None and not (set(op.nodes) & used):
                    used.update(op.nodes)
                    out.append(op)
        for i, n in enumerate(self.nodes):
            if i in used:
                continue
            op = None
            for m in (self.match_layernorm, self.match_gelu, self.match_attention, self.match_linear):
                op = m(i)
                if op is not None and not (set(op.nodes) & used):
                    break
                op = None
            if op is None:
                if n["op_type"] == "Gather" and self._weight_in(n):
                    op = FusedOp("embedding", self._data_in(n), n["output"], {"table": self._weight_in(n)[0]}, [i])
                elif n["op_type"] == "Add" and not self._weight_in(n):
                    op = FusedOp("add", n["input"], n["output"], nodes=[i])
                else:
                    op = FusedOp("other", n["input"], n["output"], nodes=[i], attrs={"op_type": n["op_type"]})
            used.update(op.nodes)
            out.append(op)
        out.sort(key=lambda o: min(o.nodes))
        return out


def name_encoder_weights(ops: List[FusedOp]) -> Dict[str, str]:
    """Canonical names for a BERT-style encoder export whose initializers carry no usable names (``onnx::MatMul_123``):
    the structure tells which weight is which. Per layer: three linears feed an attention core (query, key, value in the
    order of the core's inputs), the linear after it is the output projection, the next LayerNorm the post-attention
    norm, then up projection -> GELU -> down projection -> LayerNorm."""
    by_out = {o.outputs[0]: o for o in ops if o.outputs}

    def source_linear(value, depth=6):        # walk up through reshapes / transposes to the linear that made a tensor
        for _ in range(depth):
            o = by_out.get(value)
            if o is None:
                return None
            if o.kind == "linear":
                return o
            if not o.inputs:
                return None
            value = o.inputs[0]
        return None

    names: Dict[str, str] = {}
    layer = 0
    seq = [o for o in ops if o.kind in ("attention", "linear", "layernorm", "gelu", "embedding")]
    emb = [o for o in seq if o.kind == "embedding"]
    for o, nm in zip(emb, ("embed_tokens", "position_embeddings", "token_type_embeddings")):
        names[nm] = o.weights["table"]
    first_attn = next((i for i, o in enumerate(seq) if o.kind == "attention"), None)
    if first_attn is not None:
        ln0 = [o for o in seq[:first_attn] if o.kind == "layernorm"]
        if ln0:
            names["embed_norm"], names["embed_norm_bias"] = ln0[-1].weights.get("gamma"), ln0[-1].weights.get("beta")
    for i, o in enumerate(seq):
        if o.kind != "attention":
            continue
        p = f"L{layer}."
        for role, value in zip(("q_proj", "k_proj", "v_proj"), o.inputs):
            lin = source_linear(value)
            if lin is not None:
                names[p + role] = lin.weights["weight"]
                if lin.weights.get("bias"):
                    names[p + role + "_bias"] = lin.weights["bias"]
        rest = seq[i + 1:]
        stop = next((j for j, r in enumerate(rest) if r.kind == "attention"), len(rest))
        body = rest[:stop]
        lins = [r for r in body if r.kind == "linear"]
        if stop < len(rest):                    # the q / k / v linears of the NEXT layer sit before its attention core
            lins = lins[:-3] if len(lins) >= 6 else lins
        lns = [r for r in body if r.kind == "layernorm"]
        for role, lin in zip(("o_proj", "up_proj", "down_proj"), lins):
            names[p + role] = lin.weights["weight"]
            if lin.weights.get("bias"):
                names[p + role + "_bias"] = lin.weights["bias"]
        for role, ln in zip(("post_attn_norm", "post_ffn_norm"), lns):
            names[p + role] = ln.weights.get("gamma")
            names[p + role + "_bias"] = ln.weights.get("beta")
        layer += 1
    return {k: v for k, v in names.items() if v}


def import_graph(path):
    """-> (tensors, fused ops, canonical-name map recovered from the structure)."""
    tensors, nodes = read_onnx(path)
    ops = OnnxGraph(nodes, tensors.keys()).fuse()
    return tensors, ops, name_encoder_weights(ops)
