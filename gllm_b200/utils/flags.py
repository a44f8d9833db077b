"""Environment flags in one place (read once, typed, documented).

Reference parity: the reference's environment variables (``GLLM_CACHE_DIR``, ``HF_ENDPOINT / HF_TOKEN / HF_HOME /
HF_HUB_CACHE``, ``GLLM_DEBUG_JIT``, ``GLLM_DUMP_MEGA``, ``GLLM_DUMP_FILTER``, ``GLLM_DUMP_LAYERS``,
``GLLM_DEBUG_RESOURCE``, ``GLLM_NAN_TRAP``, ``GLLM_GUARD_SCRATCH``, ``GLLM_TRACE_SWAP``,
``GLLM_TRUNCATE_LAYERS``). JIT-specific ones map onto what exists here (kernel build verbosity, tensor dumps).
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field
from typing import List, Optional


def _b(name: str, default: bool = False) -> bool:
    v = os.environ.get(name)
    return default if v is None else v.strip().lower() in ("1", "true", "yes", "on")


def _i(name: str, default: Optional[int] = None) -> Optional[int]:
    v = os.environ.get(name)
    try:
        return int(v) if v not in (None, "") else default
    except ValueError:
        return default


@dataclass
class Flags:
    cache_dir: str = ""
    hf_endpoint: str = ""
    hf_token: Optional[str] = None
    hf_home: Optional[str] = None
    debug_build: bool = False            # GLLM_DEBUG_JIT: verbose kernel build (-Xptxas -v), per-call sync
    dump_dir: Optional[str] = None       # GLLM_DUMP_MEGA: directory for tensor dumps
    dump_filter: Optional[str] = None
    dump_layers: List[int] = field(default_factory=list)
    debug_resource: bool = False
    nan_trap: bool = False
    guard_scratch: bool = False
    trace_swap: bool = False
    truncate_layers: Optional[int] = None
    trace: bool = False
    sync_each_call: bool = False

    @staticmethod
    def from_env() -> "Flags":
        layers = [int(x) for x in os.environ.get("GLLM_DUMP_LAYERS", "").split(",") if x.strip().isdigit()]
        return Flags(
            cache_dir=os.environ.get("GLLM_CACHE_DIR", os.path.join(os.path.expanduser("~"), ".gllm", "models")),
            hf_endpoint=os.environ.get("HF_ENDPOINT", "https://huggingface.co"),
            hf_token=os.environ.get("HF_TOKEN"), hf_home=os.environ.get("HF_HOME") or os.environ.get("HF_HUB_CACHE"),
            debug_build=_b("GLLM_DEBUG_JIT"), dump_dir=os.environ.get("GLLM_DUMP_MEGA") or os.environ.get("GLLM_DUMP_DIR"),
            dump_filter=os.environ.get("GLLM_DUMP_FILTER"), dump_layers=layers, debug_resource=_b("GLLM_DEBUG_RESOURCE"),
            nan_trap=_b("GLLM_NAN_TRAP"), guard_scratch=_b("GLLM_GUARD_SCRATCH"), trace_swap=_b("GLLM_TRACE_SWAP"),
            truncate_layers=_i("GLLM_TRUNCATE_LAYERS"), trace=_b("GLLM_TRACE"), sync_each_call=_b("GLLM_SYNC_EACH_CALL"))


def apply_truncate_layers(cfg, flags: Optional[Flags] = None):
    """Debug aid: run only the first N layers of a model (changes the outputs, never used in benchmarks)."""
    flags = flags or Flags.from_env()
    if flags.truncate_layers and 0 < flags.truncate_layers < cfg.num_layers:
        cfg.num_layers = flags.truncate_layers
    return cfg
