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


class Backend:
    """What an execution backend provides to the engine (the reference's ``trait Backend``,
    src/compat/mod.rs:77-345). One implementation exists here: B200 kernels for CUDA tensors, the fp32 oracle for
    CPU tensors — both behind the same op functions, so the methods below are thin."""

    def __init__(self, detected: DetectedBackend):
        self.info = detected

    @property
    def device(self) -> torch.device:
        return self.info.device

    def alloc_kv_cache(self, model, num_pages: int):
        return model.alloc_kv_cache(num_pages)

    def gpu_sm_version(self) -> int:
        return self.info.compute_capability[0] * 10 + self.info.compute_capability[1]

    def get_memory_pressure(self) -> float:
        if self.info.device.type != "cuda":
            from ..runtime.sensors import host_memory_pressure
            return host_memory_pressure()
        free, total = torch.cuda.mem_get_info(self.info.device)
        return 1.0 - free / total

    def sample_from_tensor(self, logits, params, **kw):
        from .. import ops
        return ops.sample(logits, params, **kw)

    def quantized_matmul(self, a, qweight):
        from ..ops.quant_gemm import qgemm
        return qgemm(a, qweight)

    def dequantize(self, type_id: int, raw, n_elems: int):
        from ..loader.quant import dequantize
        return dequantize(type_id, raw, n_elems)

    def swap_out_pages(self, swap, keys):
        from ..scheduler.swap import DmaCommand
        return [swap.execute(DmaCommand.EVICT_TO_DRAM, k) for k in keys]

    def swap_in_pages(self, swap, keys):
        from ..scheduler.swap import DmaCommand
        return [swap.execute(DmaCommand.PROMOTE_TO_HBM, k) for k in keys]


class BackendContext:
    """Owns the detected backend and the executor built on it (src/backend/mod.rs:1215-1333)."""

    def __init__(self, prefer: Optional[str] = None):
        self.backend = Backend(detect_backend(prefer))
        self.executor = None
        import threading
        self.lock = threading.Lock()

    def build_executor(self, model, engine_cfg=None, tokenizer=None):
        from ..engine.executor import LLMEngine
        with self.lock:
            self.executor = LLMEngine(model, engine_cfg, tokenizer)
        return self.executor
