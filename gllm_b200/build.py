"""In-tree native build: every CUDA kernel is compiled for sm_100a with nvcc into
``gllm_b200/_lib/libgllm_kernels.so`` (plain C ABI, loaded with ctypes), and the C++ host
runtime (scheduler, CPU oracle, loaders, C FFI) into sibling shared objects.

The libraries are built next to the sources so a copy of the tree carries them; nothing is
installed into site-packages and nothing depends on a JIT cache.

Usage:  python -m gllm_b200.build [--force] [--verbose]
"""
from __future__ import annotations

import concurrent.futures as cf
import os
import shutil
import subprocess
import sys
import sysconfig
from pathlib import Path

ROOT = Path(__file__).resolve().parent
CSRC = ROOT / "csrc"
LIB = ROOT / "_lib"
OBJ = LIB / "obj"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC,-fvisibility=hidden",
    "--expt-relaxed-constexpr",
    "-diag-suppress", "550",
]
CXX_FLAGS = ["-O3", "-std=c++17", "-fPIC", "-fvisibility=hidden", "-Wall", "-Wno-unused-function", "-pthread"]


def _nvcc() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found; CUDA 12.9 toolkit is required to build the sm_100a kernels")
    return cand


def _newer(src_list, out: Path) -> bool:
    if not out.exists():
        return True
    t = out.stat().st_mtime
    return any(Path(s).stat().st_mtime > t for s in src_list)


def _run(cmd, verbose=False):
    if verbose:
        print(" ".join(str(c) for c in cmd), flush=True)
    r = subprocess.run([str(c) for c in cmd], capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"build command failed ({r.returncode}): {' '.join(str(c) for c in cmd)}\n{r.stdout}\n{r.stderr}")
    if verbose and (r.stdout or r.stderr):
        print(r.stdout, r.stderr, flush=True)
    return r


def build_kernels(force=False, verbose=False, trace=False) -> Path:
    """nvcc -> libgllm_kernels.so (all .cu files under csrc/kernels). ``trace``: a second library,
    libgllm_kernels_trace.so, compiled with -DGLLM_TRACE (phase stamps in the GEMM kernel; loaded instead of the regular
    one when GLLM_TRACE_LIB=1)."""
    LIB.mkdir(exist_ok=True)
    obj_dir = LIB / ("obj_trace" if trace else "obj")
    obj_dir.mkdir(exist_ok=True)
    out = LIB / ("libgllm_kernels_trace.so" if trace else "libgllm_kernels.so")
    srcs = sorted((CSRC / "kernels").glob("*.cu"))
    hdrs = sorted((CSRC / "kernels").glob("*.cuh")) + sorted((CSRC / "kernels").glob("*.h"))
    nvcc = _nvcc()
    objs, jobs = [], []
    for s in srcs:
        o = obj_dir / (s.stem + ".o")
        objs.append(o)
        if force or _newer([s] + hdrs, o):
            jobs.append([nvcc, *NVCC_FLAGS] + (["-DGLLM_TRACE"] if trace else []) + (["-Xptxas", "-v"] if verbose else [])
                        + ["-c", s, "-o", o])
    if jobs:
        with cf.ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            list(ex.map(lambda c: _run(c, verbose), jobs))
    if jobs or force or _newer(objs, out):
        _run([nvcc, "-shared", "-o", out, *objs, "-gencode", "arch=compute_100a,code=sm_100a"], verbose)
    return out


def _pybind_includes():
    import pybind11
    return ["-I", pybind11.get_include(), "-I", sysconfig.get_paths()["include"]]


def build_cxx_module(name: str, subdir: str, pybind=True, force=False, verbose=False, extra=()) -> Path:
    """g++ -> <name>.so from csrc/<subdir>/*.cpp (pybind11 extension module or plain C ABI library)."""
    LIB.mkdir(exist_ok=True)
    srcs = sorted((CSRC / subdir).glob("*.cpp"))
    hdrs = sorted((CSRC / subdir).glob("*.h")) + sorted((CSRC / subdir).glob("*.hpp"))
    if not srcs:
        raise RuntimeError(f"no sources under {CSRC / subdir}")
    suffix = sysconfig.get_config_var("EXT_SUFFIX") if pybind else ".so"
    out = LIB / (name + suffix)
    if force or _newer(srcs + hdrs, out):
        cmd = ["g++", *CXX_FLAGS, "-shared", "-o", out, *srcs, *extra]
        if pybind:
            cmd += _pybind_includes()
        _run(cmd, verbose)
    return out


def _python_embed_flags():
    """Compiler / linker flags to embed the running interpreter (the C ABI shim)."""
    inc = sysconfig.get_paths()["include"]
    libdir = sysconfig.get_config_var("LIBDIR") or ""
    ver = sysconfig.get_config_var("LDVERSION") or sysconfig.get_python_version()
    return ("-I", inc, "-L", libdir, f"-lpython{ver}", f"-Wl,-rpath,{libdir}")


def build_all(force=False, verbose=False):
    outs = [build_kernels(force, verbose)]
    if (LIB / "libgllm_kernels_trace.so").exists():     # keep an existing trace build in step with the sources
        outs.append(build_kernels(force, verbose, trace=True))
    for name, sub, pyb, extra in (("_sched", "sched", True, ()), ("libgllm_cpuref", "ref", False, ("-fopenmp",)),
                                  ("libgllm_loader", "loader", False, ("-fopenmp",)),
                                  ("libgllm_ffi", "ffi", False, _python_embed_flags())):
        if any((CSRC / sub).glob("*.cpp")):
            outs.append(build_cxx_module(name, sub, pybind=pyb, force=force, verbose=verbose, extra=extra))
    return outs


if __name__ == "__main__":
    force = "--force" in sys.argv
    verbose = "--verbose" in sys.argv
    for o in build_all(force, verbose):
        print("built", o)
    if "--trace" in sys.argv:
        print("built", build_kernels(force, verbose, trace=True))
