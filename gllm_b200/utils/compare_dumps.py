"""Compare two directories of dumped tensors (what GLLM_DUMP_DIR / ``engine.guard.dump_tensors`` write): per tensor
the largest absolute and relative difference and the cosine, worst first.

    python -m gllm_b200.utils.compare_dumps dir_a dir_b [--rtol 1e-2] [--atol 1e-3]

Reference parity: src/bin/compare_dumps.rs (layer-by-layer comparison of two dump directories).
"""
from __future__ import annotations

import argparse
import os
from typing import Dict, List

import torch


def compare(dir_a: str, dir_b: str, rtol: float = 1e-2, atol: float = 1e-3) -> List[Dict[str, object]]:
    names = sorted(set(os.listdir(dir_a)) & set(os.listdir(dir_b)))
    rows = []
    for n in names:
        if not n.endswith(".pt"):
            continue
        a = torch.load(os.path.join(dir_a, n), map_location="cpu", weights_only=True).float()
        b = torch.load(os.path.join(dir_b, n), map_location="cpu", weights_only=True).float()
        if a.shape != b.shape:
            rows.append({"name": n, "ok": False, "why": f"shapes {tuple(a.shape)} vs {tuple(b.shape)}", "max_abs": float("inf")})
            continue
        d = (a - b).abs()
        rel = d / b.abs().clamp_min(atol)
        cos = torch.nn.functional.cosine_similarity(a.flatten(), b.flatten(), dim=0).item() if a.numel() else 1.0
        ok = bool((d <= atol + rtol * b.abs()).all())
        rows.append({"name": n, "ok": ok, "max_abs": float(d.max()) if d.numel() else 0.0,
                     "max_rel": float(rel.max()) if rel.numel() else 0.0, "cosine": cos})
    only = sorted(set(os.listdir(dir_a)) ^ set(os.listdir(dir_b)))
    for n in only:
        rows.append({"name": n, "ok": False, "why": "present on one side only", "max_abs": float("inf")})
    rows.sort(key=lambda r: -r["max_abs"])
    return rows


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("dir_a")
    ap.add_argument("dir_b")
    ap.add_argument("--rtol", type=float, default=1e-2)
    ap.add_argument("--atol", type=float, default=1e-3)
    a = ap.parse_args(argv)
    rows = compare(a.dir_a, a.dir_b, a.rtol, a.atol)
    for r in rows:
        tail = r.get("why") or f"max_abs {r['max_abs']:.3e} max_rel {r['max_rel']:.3e} cos {r['cosine']:.6f}"
        print(f"{'ok ' if r['ok'] else 'BAD'} {r['name']:<48} {tail}")
    return 0 if all(r["ok"] for r in rows) else 1


if __name__ == "__main__":
    raise SystemExit(main())
