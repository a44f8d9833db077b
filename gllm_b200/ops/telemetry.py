"""Device-side layer telemetry and in-place KV page requantisation (``csrc/kernels/telemetry.cu``); CPU paths are
the plain tensor formulas (``runtime/epilogue.py``, ``kv_cache/quant.py``)."""
from __future__ import annotations

from typing import Optional, Sequence

import torch

from . import _native as nv
from ._native import F, I, L, P

nv.register("gllm_layer_telemetry", I, [P, P, L, P, L, F, P, P])
nv.register("gllm_kv_requant_pages", I, [P, I, L, P, I, I, I, P])

TIER_MODES = {"fp8": 1, "kivi4": 2, "kivi2": 3}


def layer_telemetry(x_in: torch.Tensor, x_out: torch.Tensor, act: Optional[torch.Tensor] = None, eps: float = 1e-3):
    """-> dict(delta_rho = ||x_out - x_in|| / ||x_in||, sparsity = fraction of |act| < eps)."""
    if not x_in.is_cuda:
        d = float((x_out.float() - x_in.float()).norm() / x_in.float().norm().clamp_min(1e-12))
        sp = float((act.float().abs() < eps).float().mean()) if act is not None else 0.0
        return {"delta_rho": d, "sparsity": sp}
    out = torch.empty(3, dtype=torch.float32, device=x_in.device)
    rc = nv.lib().gllm_layer_telemetry(x_in.data_ptr(), x_out.data_ptr(), x_in.numel(), nv.ptr(act),
                                       act.numel() if act is not None else 0, float(eps), out.data_ptr(), nv.stream_ptr())
    nv.check(rc, "layer_telemetry")
    d2, n2, z = out.tolist()
    return {"delta_rho": (d2 / max(n2, 1e-24)) ** 0.5, "sparsity": z / act.numel() if act is not None else 0.0}


def requant_pages_(cache: torch.Tensor, pages: Sequence[int], tier: str, row_len: Optional[int] = None) -> torch.Tensor:
    """Round pages of ``cache`` [num_pages, ...] (bf16 on the GPU) through ``tier`` in place."""
    mode = TIER_MODES[tier]
    row_len = row_len or cache.shape[-1]
    page_elems = cache[0].numel()
    if not cache.is_cuda:
        for p in pages:
            x = cache[p].float()
            if mode == 1:
                s = x.abs().amax().clamp_min(1e-12) / 448.0
                cache[p] = ((x / s).to(torch.float8_e4m3fn).float() * s).to(cache.dtype)
            else:
                lv = 15 if mode == 2 else 3
                r = x.reshape(-1, row_len)
                lo, hi = r.amin(1, keepdim=True), r.amax(1, keepdim=True)
                sc = (hi - lo).clamp_min(1e-8) / lv
                cache[p] = (torch.round((r - lo) / sc).clamp(0, lv) * sc + lo).reshape(cache[p].shape).to(cache.dtype)
        return cache
    ids = torch.tensor(list(pages), dtype=torch.int32, device=cache.device)
    rc = nv.lib().gllm_kv_requant_pages(cache.data_ptr(), cache.shape[0], page_elems, ids.data_ptr(), ids.numel(), row_len, mode,
                                        nv.stream_ptr())
    nv.check(rc, "kv_requant_pages")
    return cache
