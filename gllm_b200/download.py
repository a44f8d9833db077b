"""Model download CLI.

    python -m gllm_b200.download <model-id> [--source hf|modelscope] [--file-filter PATTERN] [--cache-dir DIR]

Reference parity: src/bin/download.rs (download CLI over the loader's hub resolution).
"""
from __future__ import annotations

import argparse
import sys


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="gllm_b200.download")
    ap.add_argument("model_id")
    ap.add_argument("--source", choices=["hf", "modelscope"], default="hf")
    ap.add_argument("--file-filter", default=None, help="only files whose name contains this (e.g. Q4_K_M)")
    ap.add_argument("--cache-dir", default=None)
    a = ap.parse_args(argv)
    from pathlib import Path
    from .loader.hub import resolve_model
    from .loader.loader import LoaderConfig
    cfg = LoaderConfig(source="huggingface" if a.source == "hf" else "modelscope", gguf_file_filter=a.file_filter)
    if a.cache_dir:
        cfg.cache_dir = Path(a.cache_dir)
    try:
        path = resolve_model(a.model_id, cfg)
    except Exception as exc:
        print(f"download failed: {exc}", file=sys.stderr)
        return 1
    print(path)
    return 0


if __name__ == "__main__":
    sys.exit(main())
