"""Session / prefix-cache persistence: snapshot the KV pages that back finished sessions to a file and load them
into a fresh engine, so a restarted server answers the next turn of a conversation without recomputing its
history.

Reference parity: session KV resume (src/engine/executor_api.rs:411-469, src/scheduler/memory_manager.rs:582-720)
keeps finalised positions in memory only; the snapshot file is this build's addition for restarts
(model weights themselves are reloaded from their checkpoint formats).
"""
from __future__ import annotations

from typing import Dict, List

import torch

FORMAT_VERSION = 1


def save_sessions(engine, path: str) -> Dict[str, int]:
    """Writes {session id: tokens, per-layer page contents} for every session whose pages are still cached."""
    b = engine.batcher
    out = {"version": FORMAT_VERSION, "page_size": 16, "layers": len(engine.kv_caches),
           "page_shape": tuple(engine.kv_caches[0].shape[1:]), "dtype": str(engine.kv_caches[0].dtype), "sessions": {}}
    saved = {}
    for sid in b.session_ids():
        toks = list(b.session_tokens(sid))
        pages = list(b.lookup_prefix_pages(toks))
        if not pages:
            continue
        idx = torch.tensor(pages, dtype=torch.long, device=engine.kv_caches[0].device)
        data = torch.stack([c.index_select(0, idx) for c in engine.kv_caches]).cpu()    # [L, n_pages, ...]
        out["sessions"][sid] = {"tokens": toks[: len(pages) * 16], "kv": data}
        saved[sid] = len(pages) * 16
    torch.save(out, path)
    return saved


def load_sessions(engine, path: str) -> Dict[str, int]:
    """Restores sessions into ``engine`` (same model geometry). Returns {session id: tokens restored}."""
    snap = torch.load(path, map_location="cpu", weights_only=True)     # tensors, lists, dicts and scalars only
    if snap.get("version") != FORMAT_VERSION:
        raise ValueError("unknown session snapshot version")
    if tuple(snap["page_shape"]) != tuple(engine.kv_caches[0].shape[1:]) or snap["layers"] != len(engine.kv_caches):
        raise ValueError("session snapshot does not match this model's KV geometry")
    restored = {}
    for sid, rec in snap["sessions"].items():
        pages = list(engine.batcher.import_prefix([int(t) for t in rec["tokens"]], sid))
        kv = rec["kv"]
        n = 0
        for i, p in enumerate(pages):
            n += 1
            if p < 0:
                continue                     # that page was already cached (shared prefix)
            for l, cache in enumerate(engine.kv_caches):
                cache[p].copy_(kv[l, i].to(cache.device, cache.dtype))
        restored[sid] = n * 16
    return restored
