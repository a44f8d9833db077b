"""Model resolution and download: local cache -> Hugging Face hub -> ModelScope.

Reference parity: ``hf_hub.rs`` / ``modelscope.rs`` / ``downloader.rs`` — ``HF_ENDPOINT`` / ``HF_TOKEN`` /
``HF_HOME`` / ``HF_HUB_CACHE``, chunked downloads that resume from a partial file, fallback to the other hub,
``~/.gllm/models`` cache (src/loader/fragments/types.inc.rs:133-176). With no network (or
``HF_HUB_OFFLINE=1``) only the caches are consulted and a miss raises ``ModelNotFound``.
"""
from __future__ import annotations

import hashlib
import json
import os
import urllib.error
import urllib.request
from pathlib import Path
from typing import Iterable, List, Optional

WEIGHT_PATTERNS = (".safetensors", ".gguf", ".gllm", ".bin", ".onnx", ".json", ".model", ".txt")


def hf_cache_dirs() -> List[Path]:
    out = []
    if os.environ.get("HF_HUB_CACHE"):
        out.append(Path(os.environ["HF_HUB_CACHE"]))
    home = Path(os.environ.get("HF_HOME", Path.home() / ".cache" / "huggingface"))
    out.append(home / "hub")
    return out


def find_in_caches(model_id: str, cache_dir: Path) -> Optional[Path]:
    flat = model_id.replace("/", "--")
    own = cache_dir / flat
    if own.exists() and any(own.iterdir()):
        return own
    for hub in hf_cache_dirs():
        snaps = hub / f"models--{flat}" / "snapshots"
        if snaps.exists():
            revs = sorted(snaps.iterdir(), key=lambda p: p.stat().st_mtime, reverse=True)
            if revs:
                return revs[0]
    ms = Path(os.environ.get("MODELSCOPE_CACHE", Path.home() / ".cache" / "modelscope")) / "hub" / model_id
    if ms.exists():
        return ms
    return None


def _request(url: str, headers=None, start: int = 0):
    h = dict(headers or {})
    if start:
        h["Range"] = f"bytes={start}-"
    return urllib.request.urlopen(urllib.request.Request(url, headers=h), timeout=30)


def download_file(url: str, dest: Path, headers=None, chunk: int = 8 << 20, sha256: Optional[str] = None) -> Path:
    """Chunked download that resumes from ``dest.part``; optional checksum."""
    dest.parent.mkdir(parents=True, exist_ok=True)
    part = dest.with_suffix(dest.suffix + ".part")
    start = part.stat().st_size if part.exists() else 0
    with _request(url, headers, start) as r, open(part, "ab" if start else "wb") as f:
        if start and r.status != 206:  # server ignored the range: start over
            f.truncate(0)
        while True:
            b = r.read(chunk)
            if not b:
                break
            f.write(b)
    if sha256:
        h = hashlib.sha256()
        with open(part, "rb") as f:
            for b in iter(lambda: f.read(1 << 20), b""):
                h.update(b)
        if h.hexdigest() != sha256:
            part.unlink()
            raise IOError(f"checksum mismatch for {url}")
    part.rename(dest)
    return dest


def list_hf_files(model_id: str, endpoint: str, token: Optional[str]) -> List[dict]:
    headers = {"Authorization": f"Bearer {token}"} if token else {}
    with _request(f"{endpoint}/api/models/{model_id}", headers) as r:
        info = json.loads(r.read().decode())
    return info.get("siblings", [])


def download_from_hf(model_id: str, dest: Path, file_filter=None) -> Path:
    endpoint = os.environ.get("HF_ENDPOINT", "https://huggingface.co").rstrip("/")
    token = os.environ.get("HF_TOKEN")
    headers = {"Authorization": f"Bearer {token}"} if token else {}
    for sib in list_hf_files(model_id, endpoint, token):
        name = sib["rfilename"]
        if not name.endswith(WEIGHT_PATTERNS) or (file_filter and not file_filter(name)):
            continue
        download_file(f"{endpoint}/{model_id}/resolve/main/{name}", dest / name, headers)
    return dest


def download_from_modelscope(model_id: str, dest: Path, file_filter=None) -> Path:
    base = os.environ.get("MODELSCOPE_ENDPOINT", "https://modelscope.cn").rstrip("/")
    with _request(f"{base}/api/v1/models/{model_id}/repo/files?Recursive=true") as r:
        files = json.loads(r.read().decode()).get("Data", {}).get("Files", [])
    for f in files:
        name = f.get("Path", "")
        if f.get("Type") == "tree" or not name.endswith(WEIGHT_PATTERNS) or (file_filter and not file_filter(name)):
            continue
        download_file(f"{base}/api/v1/models/{model_id}/repo?FilePath={name}", dest / name, sha256=f.get("Sha256") or None)
    return dest


def resolve_model(model_id: str, cfg) -> Path:
    from .loader import ModelNotFound
    hit = find_in_caches(model_id, Path(cfg.cache_dir))
    if hit is not None:
        return hit
    if cfg.offline:
        raise ModelNotFound(f"{model_id}: not in {cfg.cache_dir} or the Hugging Face cache, and offline mode is set")
    dest = Path(cfg.cache_dir) / model_id.replace("/", "--")
    flt = None
    if cfg.gguf_file_filter:
        import re
        rx = re.compile(cfg.gguf_file_filter, re.I)
        flt = lambda n: (not n.endswith(".gguf")) or bool(rx.search(n))
    order = [download_from_hf, download_from_modelscope] if cfg.source == "huggingface" else \
        [download_from_modelscope, download_from_hf]
    if not cfg.fallback:
        order = order[:1]
    errors = []
    for fn in order:
        try:
            return fn(model_id, dest, flt)
        except (urllib.error.URLError, OSError, ValueError, KeyError) as e:
            errors.append(f"{fn.__name__}: {e}")
    raise ModelNotFound(f"{model_id}: could not be downloaded ({'; '.join(errors)})")
