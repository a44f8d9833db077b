"""ctypes binding to ``libgllm_kernels.so`` (the hand-written sm_100a kernels).

The library is mandatory whenever a CUDA tensor reaches an op: a missing or stale library is an
error, never a silent fallback to PyTorch. CPU tensors take the PyTorch reference path, which is
also the numerical oracle used by the tests.
"""
from __future__ import annotations

import ctypes
import threading
from ctypes import c_float, c_int, c_longlong, c_ulonglong, c_void_p
from pathlib import Path

_LIB_DIR = Path(__file__).resolve().parent.parent / "_lib"
_lock = threading.Lock()
_lib = None

P, I, L, F, U = c_void_p, c_int, c_longlong, c_float, c_ulonglong

_SIGNATURES = {
    "gllm_last_error": (ctypes.c_char_p, []),
    "gllm_error_word": (P, []),
    "gllm_set_error_word": (I, [P]),
    "gllm_check_error": (I, []),
    "gllm_sm_count": (I, []),
    "gllm_kernels_abi_version": (I, []),
    "gllm_gemm_bf16": (I, [P, L, P, L, P, L, I, I, I, I, P, P, I, F, F, I, P, I, I]),
    "gllm_gemm_bf16_softcap": (I, [P, L, P, L, P, L, I, I, I, I, P, P, I, F, F, I, P, F]),
    "gllm_gemm_set_splitk_workspace": (I, [P, L, P, I]),
    "gllm_gemm_set_splitk_workspace_stream": (I, [P, P, L, P, I]),
    "gllm_gemm_bf16_residual": (I, [P, L, P, L, P, L, P, L, P, I, I, I, P, I, P, I, I]),
    "gllm_gemm_set_pair": (I, [I, I]),
    "gllm_gemm_set_pair_big_m": (I, [I]),
    "gllm_gemm_bf16_residual_allreduce": (I, [P, L, P, L, P, L, P, L, P, I, I, I, P, I, P, I, I, I, I, P, P, P, P, P, L]),
    "gllm_gemm_bf16_residual_allreduce_push": (I, [P, L, P, L, P, L, P, I, I, I, P, I, P, I, I, P, P, L, L, L, L, L, L, P]),
    "gllm_gemm_bf16_residual_allreduce_ll": (I, [P, L, P, L, P, L, P, I, I, I, P, I, P, I, I, P, P, L, L, L, L, L, P]),
    "gllm_gemm_bf16_residual_reduce_scatter": (I, [P, L, P, L, P, L, P, I, I, I, P, P, I, I, P, L, L, L, P]),
    "gllm_gemm_set_block_rows": (I, [P]),
    "gllm_gemm_set_allgather_input": (I, [P, L, P, L, I, I, P, P, L, L, L, P, P]),
    "gllm_set_option": (L, [ctypes.c_char_p, L]),
    "gllm_get_option": (L, [ctypes.c_char_p]),
    "gllm_gemm_trace_enabled": (I, []),
    "gllm_gemm_bf16_glu": (I, [P, L, P, L, P, L, I, I, I, I, P, I, F, F, I, P, I, P, I, I]),
    "gllm_gemm_bf16_grouped": (I, [P, L, P, L, P, L, I, I, I, P, I, I, P, I]),
    "gllm_gemm_bf16_qkv": (I, [P, L, P, L, I, I, I, I, P, P, I, P, P, P, P, I, P, P, F, P, I, F, F, P, P, I, I]),
    "gllm_gemm_bf16_qkv_fp8kv": (I, [P, L, P, L, I, I, I, I, P, P, I, P, P, P, P, I, P, P, F, P, I, F, F, P, F, P, I, I]),
    "gllm_gemm_fp8": (I, [P, L, P, L, P, L, I, I, I, I, P, P, I, P, I, I]),
    "gllm_decode_scratch_floats": (L, [I, I, I]),
    "gllm_paged_decode": (I, [P, P, P, I, P, I, P, I, I, I, F, I, I, P, P, I, P, P]),
    "gllm_paged_prefill": (I, [P, P, P, I, P, I, P, P, P, I, I, I, I, F, I, I, P, P]),
    "gllm_paged_prefill_tc": (I, [P, P, P, I, P, I, P, P, P, I, I, I, I, I, F, I, I, P, P]),
    "gllm_paged_decode_fp8": (I, [P, P, P, I, P, I, P, I, I, I, F, I, I, P, P, I, P, F, P]),
    "gllm_paged_prefill_fp8": (I, [P, P, P, I, P, I, P, P, P, I, I, I, I, F, I, I, P, F, P]),
    "gllm_embed_gather": (I, [P, P, I, I, F, P, P, I, P]),
    "gllm_rmsnorm": (I, [P, P, P, I, I, F, I, P, P, P, P]),
    "gllm_layernorm": (I, [P, P, P, P, I, I, F, P, P]),
    "gllm_glu": (I, [P, L, I, I, I, P, P]),
    "gllm_rope_kv_write": (I, [P, L, I, I, I, I, I, P, P, P, P, I, P, P, F, P, P, I, P]),
    "gllm_paged_attention_generic": (I, [P, P, P, I, P, I, P, P, P, I, I, I, I, I, F, I, I, P]),
    "gllm_paged_attention_fp8kv": (I, [P, P, P, I, P, I, P, P, P, I, I, I, I, I, F, I, I, F, P]),
    "gllm_rope_kv_write_fp8": (I, [P, L, I, I, I, I, I, P, P, P, P, I, P, P, F, P, P, I, F, P]),
    "gllm_pool": (I, [P, P, P, I, I, I, P, P]),
    "gllm_sample": (I, [P, L, I, I, I, P, U, P, P, P, P]),
    "gllm_argmax": (I, [P, L, I, I, I, P, P, P]),
}

_OPTIONAL = set()


class NativeLibraryError(RuntimeError):
    pass


def lib_path() -> Path:
    import os
    if os.environ.get("GLLM_TRACE_LIB") == "1":      # the -DGLLM_TRACE build (python -m gllm_b200.build --trace)
        return _LIB_DIR / "libgllm_kernels_trace.so"
    return _LIB_DIR / "libgllm_kernels.so"


def available() -> bool:
    return lib_path().exists()


def lib():
    """Load (once) and return the kernel library; raises NativeLibraryError if it is not built."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        path = lib_path()
        if not path.exists():
            raise NativeLibraryError(
                f"{path} is missing: run `python -m gllm_b200.build` (needs nvcc) before using CUDA tensors")
        handle = ctypes.CDLL(str(path))
        for name, (res, args) in _SIGNATURES.items():
            try:
                fn = getattr(handle, name)
            except AttributeError:
                if name in _OPTIONAL:
                    continue
                raise NativeLibraryError(f"{path} is stale: symbol {name} not found; rebuild with --force")
            fn.restype = res
            fn.argtypes = args
        _lib = handle
        _apply_env_options(handle)
    return _lib


# Environment variables that map onto library settings (read once, when the library is loaded). The native code itself
# reads no environment variable.
_ENV_OPTIONS = (
    ("GLLM_PDL", "pdl", int), ("GLLM_AR_SPLIT", "ar_split", int), ("GLLM_QKV_TWO_ROWS", "qkv_two_rows", int), ("GLLM_PREFILL_TC", "prefill_tc", int), ("GLLM_DEC_TILES", "dec_tiles", int),
    ("GLLM_AR_TWO_SHOT", "ar_two_shot", int), ("GLLM_PAIR_MAX_M", "pair_max_m", int), ("GLLM_PAIR_BIG_M", "pair_big_m", int),
    ("GLLM_WAIT_NS", "wait_ns", int), ("GLLM_PEER_WAIT_NS", "peer_wait_ns", int),
)


def _apply_env_options(handle):
    import os
    env = os.environ
    for var, name, conv in _ENV_OPTIONS:
        if env.get(var, "") != "":
            handle.gllm_set_option(name.encode(), conv(env[var]))
    if env.get("GLLM_NO_PARK") == "1":
        handle.gllm_set_option(b"park", 0)
    if env.get("GLLM_NO_CLUSTER_SK") == "1":
        handle.gllm_set_option(b"cluster_sk", 0)
    pair = env.get("GLLM_PAIR")          # "0": no CTA pairs anywhere; "1": every epilogue at decode sizes
    if pair == "0":
        handle.gllm_set_option(b"pair_max_m", 0)
        handle.gllm_set_option(b"pair_big_m", 0)
    elif pair == "1":
        handle.gllm_set_option(b"pair_epi_mask", 0xF)


def set_option(name: str, value: int) -> int:
    """Set a library setting (``RuntimeSettings`` in csrc/kernels/common.cuh); returns the previous value."""
    old = int(lib().gllm_set_option(name.encode(), int(value)))
    if old == -(1 << 63):
        raise KeyError(f"unknown kernel-library option {name!r}")
    return old


def get_option(name: str) -> int:
    v = int(lib().gllm_get_option(name.encode()))
    if v == -(1 << 63):
        raise KeyError(f"unknown kernel-library option {name!r}")
    return v


def set_wait_limits_ns(local_ns: int = None, peer_ns: int = None):
    """Limits of the kernels' bounded waits (on-chip barriers / flags written by another GPU). Returns the old pair."""
    old = (get_option("wait_ns"), get_option("peer_wait_ns"))
    if local_ns is not None:
        set_option("wait_ns", local_ns)
    if peer_ns is not None:
        set_option("peer_wait_ns", peer_ns)
    return old


def register(name, restype, argtypes, optional=False):
    """Let other op modules declare entry points that live in the same library."""
    _SIGNATURES[name] = (restype, argtypes)
    if optional:
        _OPTIONAL.add(name)
    if _lib is not None:
        fn = getattr(_lib, name)
        fn.restype, fn.argtypes = restype, argtypes


CALLS = [0]  # number of kernel-launching entry points called so far (bench.py reports launches)


_SYNC_EACH_CALL = __import__("os").environ.get("GLLM_SYNC_EACH_CALL", "0") == "1"


def check(rc: int, what: str):
    CALLS[0] += 1
    if rc != 0:
        msg = lib().gllm_last_error().decode("utf-8", "replace")
        raise RuntimeError(f"{what} failed: {msg}")
    if _SYNC_EACH_CALL:  # debugging aid: attribute an asynchronous fault to the call that caused it
        import torch
        try:
            torch.cuda.synchronize()
        except RuntimeError as e:
            raise RuntimeError(f"{what}: device fault surfaced right after this call: {e}") from e


def device_error() -> int:
    """Read-and-clear the device error word (synchronises). 0 means no kernel reported a problem."""
    return int(lib().gllm_check_error())


ERROR_NAMES = {
    0: "ok", 1: "timeout waiting for a TMA stage", 2: "timeout waiting for a free smem stage",
    3: "timeout waiting for an accumulator", 4: "timeout waiting for a free accumulator slot",
    5: "timeout waiting for a peer rank", 6: "page id outside the pool", 7: "expert id out of range",
    8: "timeout waiting for another CTA", 9: "bad argument",
}


_err_tensors = {}


def error_word_tensor(device):
    """The device's error word as a torch int32 tensor (allocated once per device and registered with the library),
    so that an engine can copy it to pinned memory on its own stream next to the step's results. Call it before any
    CUDA graph is captured: kernels captured earlier keep reporting to the previous word."""
    import torch
    idx = device.index if device.index is not None else torch.cuda.current_device()
    t = _err_tensors.get(idx)
    if t is None:
        with torch.cuda.device(idx):
            t = torch.zeros(16, dtype=torch.int32, device=device)
            if lib().gllm_set_error_word(t.data_ptr()) != 0:
                raise RuntimeError("could not register the error word")
        _err_tensors[idx] = t
    return t


class DeviceStatusError(RuntimeError):
    """A kernel reported a bounded-wait timeout or a bad index through the device status word."""

    def __init__(self, code: int, where: str = ""):
        self.code = code
        super().__init__(f"device kernel reported status {code} ({ERROR_NAMES.get(code, '?')}) {where}".rstrip())


def raise_on_device_error(where: str = ""):
    code = device_error()
    if code != 0:
        raise RuntimeError(f"device kernel reported status {code} ({ERROR_NAMES.get(code, '?')}) {where}")


_splitk_ws = {}


def ensure_splitk_workspace(device, scratch_floats: int = 64 << 20, num_counters: int = 8192):
    """Allocate (once per device) and register the scratch that split-K GEMMs reduce through. Every stream without a
    workspace of its own shares it, so their split-K GEMMs must not overlap; ``stream_splitk_workspace`` gives a stream
    its own."""
    import torch
    idx = device.index if device.index is not None else torch.cuda.current_device()
    if idx in _splitk_ws:
        return _splitk_ws[idx]
    with torch.cuda.device(idx):
        scratch = torch.empty(scratch_floats, dtype=torch.float32, device=device)
        counters = torch.zeros(num_counters, dtype=torch.int32, device=device)
        rc = lib().gllm_gemm_set_splitk_workspace(scratch.data_ptr(), scratch_floats, counters.data_ptr(), num_counters)
        if rc != 0:
            raise RuntimeError("could not register the split-K workspace")
    _splitk_ws[idx] = (scratch, counters)
    return _splitk_ws[idx]


_stream_ws = {}


def stream_splitk_workspace(stream, scratch_floats: int = 32 << 20, num_counters: int = 8192):
    """Give ``stream`` (a torch.cuda.Stream) its own split-K scratch and barrier words: GEMMs launched on it, or
    captured into a graph on it, then never share a partial-sum buffer or a grid barrier with GEMMs of other streams
    (a prefill stream next to the decode graphs, for instance)."""
    import torch
    key = (stream.device.index, stream.cuda_stream)
    if key in _stream_ws:
        return _stream_ws[key]
    with torch.cuda.device(stream.device):
        scratch = torch.empty(scratch_floats, dtype=torch.float32, device=stream.device)
        counters = torch.zeros(num_counters, dtype=torch.int32, device=stream.device)
        check(lib().gllm_gemm_set_splitk_workspace_stream(stream.cuda_stream, scratch.data_ptr(), scratch_floats,
                                                         counters.data_ptr(), num_counters), "gemm_set_splitk_workspace_stream")
    _stream_ws[key] = (scratch, counters)
    return _stream_ws[key]


def ptr(t):
    """Device/host pointer of a tensor or None."""
    return None if t is None else t.data_ptr()


def stream_ptr():
    import torch
    return torch.cuda.current_stream().cuda_stream
