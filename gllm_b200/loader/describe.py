"""What is in a checkpoint file: tensors (name, type, shape, bytes) and metadata, for GGUF, SafeTensors and .gllm.

    python -m gllm_b200.loader.describe model.gguf [--tensors] [--keys] [--filter substring] [--json]

Reference parity: the inspection examples of the reference (examples/gguf_inspect.rs, list_gguf_keys.rs,
list_gguf_tensors.rs, gguf_tensors.rs, list_qwen3_tensors.rs).
"""
from __future__ import annotations

import argparse
import json
from pathlib import Path
from typing import Any, Dict, List


def describe(path) -> Dict[str, Any]:
    """{"format", "metadata": {...}, "tensors": [{"name", "type", "shape", "bytes"}], "quant_types": {type: count}}."""
    p = Path(path)
    suffix = p.suffix.lower()
    out: Dict[str, Any] = {"path": str(p), "metadata": {}, "tensors": []}
    if suffix == ".gguf":
        from .gguf import GgufFile
        f = GgufFile(p)
        out["format"] = f"gguf v{f.version}"
        out["metadata"] = {k: (v if not isinstance(v, (list, tuple)) or len(v) <= 8 else f"[{len(v)} items]")
                           for k, v in f.metadata.items()}
        out["tensors"] = [{"name": n, "type": ti.type_name, "shape": list(ti.shape), "bytes": int(ti.n_bytes)}
                          for n, ti in f.tensors.items()]
    elif suffix == ".safetensors":
        from .safetensors import SafeTensorsModel
        m = SafeTensorsModel(p)
        out["format"] = "safetensors"
        for n in m.keys():
            dt, shape = m.meta(n)
            numel = 1
            for d in shape:
                numel *= int(d)
            import torch
            size = torch.empty(0, dtype=dt).element_size() if isinstance(dt, torch.dtype) else 0
            out["tensors"].append({"name": n, "type": str(dt).replace("torch.", ""), "shape": [int(d) for d in shape],
                                   "bytes": numel * size})
        cfg = m.gllm_config()
        if cfg:
            out["metadata"] = cfg
    elif suffix == ".gllm":
        from .gllm_format import GllmFile
        f = GllmFile(p)
        out["format"] = "gllm"
        out["metadata"] = dict(getattr(f, "metadata", {}) or {})
        out["tensors"] = [{"name": n, "type": str(kind).replace("torch.", ""), "shape": list(shape), "bytes": int(nbytes)}
                          for n, (kind, shape, _off, nbytes) in f.entries.items()]
    else:
        raise ValueError(f"{p}: expected a .gguf, .safetensors or .gllm file")
    types: Dict[str, int] = {}
    for t in out["tensors"]:
        types[t["type"]] = types.get(t["type"], 0) + 1
    out["quant_types"] = types
    out["total_bytes"] = sum(t["bytes"] for t in out["tensors"])
    return out


def main(argv: List[str] = None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("file")
    ap.add_argument("--tensors", action="store_true", help="list every tensor")
    ap.add_argument("--keys", action="store_true", help="list the metadata keys and values")
    ap.add_argument("--filter", default="", help="only tensors / keys containing this substring")
    ap.add_argument("--json", action="store_true")
    a = ap.parse_args(argv)
    d = describe(a.file)
    if a.filter:
        d["tensors"] = [t for t in d["tensors"] if a.filter in t["name"]]
        d["metadata"] = {k: v for k, v in d["metadata"].items() if a.filter in k}
    if a.json:
        print(json.dumps(d, default=str))
        return 0
    print(f"{d['path']}: {d['format']}, {len(d['tensors'])} tensors, {d['total_bytes'] / 2**20:.1f} MiB, types {d['quant_types']}")
    if a.keys:
        for k, v in d["metadata"].items():
            print(f"  {k} = {v}")
    if a.tensors:
        for t in d["tensors"]:
            print(f"  {t['name']:<56} {t['type']:<8} {str(t['shape']):<24} {t['bytes']}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
