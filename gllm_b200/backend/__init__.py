"""Backend detection. The reference probes CUDA -> ROCm -> Metal -> CPU and takes the first that works
(src/backend/detection.rs:47-132). This engine is written for one target, B200 (sm_100a): a CUDA device of
compute capability 10.x runs the hand-written kernels; anything else is the CPU oracle path.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch


@dataclass
class DetectedBackend:
    name: str            # "cuda-sm100" | "cpu"
    device: torch.device
    sm_count: int = 0
    compute_capability: tuple = (0, 0)
    total_memory: int = 0
    native_kernels: bool = False


def detect_backend(prefer: Optional[str] = None) -> DetectedBackend:
    if prefer in (None, "cuda", "auto") and torch.cuda.is_available():
        idx = torch.cuda.current_device()
        p = torch.cuda.get_device_properties(idx)
        cc = (p.major, p.minor)
        if cc[0] != 10:
            raise RuntimeError(f"GPU {p.name} is sm_{cc[0]}{cc[1]}; the kernels in this build are sm_100a only")
        from ..ops import _native
        _native.lib()  # fail loudly when the kernel library is missing on a GPU box
        return DetectedBackend("cuda-sm100", torch.device("cuda", idx), p.multi_processor_count, cc, p.total_memory, True)
    if prefer == "cuda":
        raise RuntimeError("CUDA backend requested but no CUDA device is available")
    return DetectedBackend("cpu", torch.device("cpu"))
