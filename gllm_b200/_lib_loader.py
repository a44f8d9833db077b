"""Import helper for the in-tree native modules under ``gllm_b200/_lib``; builds them on first use."""
from __future__ import annotations

import importlib.util
import sysconfig
from pathlib import Path

_LIB = Path(__file__).resolve().parent / "_lib"
_cache = {}


def load_ext(name: str, subdir: str):
    """Load the pybind11 extension ``_lib/<name><EXT_SUFFIX>`` (compiling csrc/<subdir> if absent)."""
    if name in _cache:
        return _cache[name]
    path = _LIB / (name + sysconfig.get_config_var("EXT_SUFFIX"))
    if not path.exists():
        from . import build
        build.build_cxx_module(name, subdir, pybind=True)
    spec = importlib.util.spec_from_file_location(name, str(path))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    _cache[name] = mod
    return mod


def shared_lib_path(name: str, subdir: str) -> Path:
    """Path of the plain C-ABI library ``_lib/<name>.so`` (compiling csrc/<subdir> if absent)."""
    path = _LIB / (name + ".so")
    if not path.exists():
        from . import build
        build.build_cxx_module(name, subdir, pybind=False, extra=("-fopenmp",))
    return path
