"""Guarded host buffers, NaN traps and tensor dumps for debugging.

Reference parity: ``MmapGuardedBuffer`` with PROT_NONE pages on both sides of the scratchpad / KV
(src/engine/mega_kernel/executor_core.inc.rs:54-160), NaN trap and dumps (:957-968). Device buffers get canary
regions that are checked on demand (a device write past the end lands in the canary, not in another tensor).
"""
from __future__ import annotations

import ctypes
import mmap
import os
from typing import Dict, Optional

import torch

_PAGE = mmap.PAGESIZE
_libc = ctypes.CDLL(None, use_errno=True)
_PROT_NONE = 0


class GuardedHostBuffer:
    """``size`` usable bytes with an inaccessible page before and after; touching a guard page faults the
    process at the faulting instruction instead of corrupting a neighbour."""

    def __init__(self, size: int):
        self.size = size
        body = (size + _PAGE - 1) // _PAGE * _PAGE
        self._map = mmap.mmap(-1, body + 2 * _PAGE, flags=mmap.MAP_PRIVATE | mmap.MAP_ANONYMOUS)
        base = ctypes.addressof(ctypes.c_char.from_buffer(self._map))
        self._base = base
        for off in (0, _PAGE + body):
            if _libc.mprotect(ctypes.c_void_p(base + off), ctypes.c_size_t(_PAGE), _PROT_NONE) != 0:
                raise OSError(ctypes.get_errno(), "mprotect failed")
        self.address = base + _PAGE
        self.view = memoryview(self._map)[_PAGE:_PAGE + size]

    def guard_addresses(self):
        body = (self.size + _PAGE - 1) // _PAGE * _PAGE
        return self._base, self._base + _PAGE + body

    def tensor(self, dtype=torch.uint8) -> torch.Tensor:
        return torch.frombuffer(self.view, dtype=dtype)


class CanaryDeviceBuffer:
    """Device tensor with ``canary`` elements of a known pattern on both sides."""
    PATTERN = 0x5A

    def __init__(self, numel: int, dtype, device, canary_bytes: int = 256):
        esz = torch.empty((), dtype=dtype).element_size()
        self.pad = canary_bytes
        self.raw = torch.full((numel * esz + 2 * canary_bytes,), self.PATTERN, dtype=torch.uint8, device=device)
        self.data = self.raw[canary_bytes:canary_bytes + numel * esz].view(dtype)
        self.data.zero_()

    def intact(self) -> bool:
        return bool((self.raw[:self.pad] == self.PATTERN).all() and (self.raw[-self.pad:] == self.PATTERN).all())


class NanTrap:
    """Checks named tensors for NaN / Inf; raises with the first offender (debug builds of a forward)."""

    def __init__(self, enabled: Optional[bool] = None, dump_dir: Optional[str] = None):
        self.enabled = (os.environ.get("GLLM_NAN_TRAP", "0") == "1") if enabled is None else enabled
        self.dump_dir = dump_dir or os.environ.get("GLLM_DUMP_DIR")
        self.checked = 0

    def check(self, name: str, t: torch.Tensor):
        if not self.enabled:
            return
        self.checked += 1
        bad = ~torch.isfinite(t.float())
        if bad.any():
            idx = torch.nonzero(bad)[0].tolist()
            if self.dump_dir:
                dump_tensors({name: t}, self.dump_dir)
            raise FloatingPointError(f"{name}: non-finite value at {idx} ({int(bad.sum())} in total)")


def dump_tensors(tensors: Dict[str, torch.Tensor], directory: str):
    os.makedirs(directory, exist_ok=True)
    for name, t in tensors.items():
        torch.save(t.detach().cpu(), os.path.join(directory, name.replace("/", "_") + ".pt"))


def nan_check_callback(trap: "NanTrap"):
    """A layer callback that runs the trap on the residual stream after every layer (debug serving: the first layer
    that produces a non-finite value is named in the exception)."""
    from .callbacks import CallbackResult, LayerCallback

    class _NanCheck(LayerCallback):
        priority = 100
        layers = None

        def post_layer(self, layer, hidden):
            trap.check(f"hidden after layer {layer}", hidden)
            return CallbackResult()
    return _NanCheck()
