"""Gemma-family specifics that the Llama-style template does not have: weightless query/key norm, value norm,
per-layer RoPE base selection (dual RoPE), LAuReL low-rank residual, AltUp predict / correct / inject, and
per-layer embeddings (PLE).

Reference parity: ``QkNorm`` (weightless L2 * sqrt(d)), ``ValueNorm`` (weightless RMS)
(src/arch/auto_graph_fragments/build_graph.inc.rs:1692-1731), ``DualRoPE`` with the per-layer base
``(layer + 1) % 5 == 0`` -> global (:1751-1754), LAuReL ``/ sqrt(2)`` residual (:1811-1846), ``AltUpPredict /
AltUpCorrect / AltUpInject`` and the PLE gather (:695,:1064,:1115). Plain tensor math: these run on any device and
are their own oracle; only the E2B / E4B checkpoints use them.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional, Tuple

import torch


def qk_norm_weightless(x: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    """x [..., heads, d] -> x / ||x||_2 * sqrt(d) (unit RMS per head, no learned weight)."""
    d = x.shape[-1]
    return (x.float() * torch.rsqrt(x.float().pow(2).sum(-1, keepdim=True) + eps * d) * math.sqrt(d)).to(x.dtype)


def value_norm(v: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    """Weightless RMS norm of the value heads."""
    return (v.float() * torch.rsqrt(v.float().pow(2).mean(-1, keepdim=True) + eps)).to(v.dtype)


def layer_uses_global_rope(layer: int, period: int = 5) -> bool:
    """Every ``period``-th layer attends globally with the large RoPE base; the rest are sliding-window layers
    with the local base."""
    return (layer + 1) % period == 0


def dual_rope_theta(layer: int, global_theta: float, local_theta: float, period: int = 5) -> float:
    return global_theta if layer_uses_global_rope(layer, period) else local_theta


def build_dual_rope_tables(cfg, max_pos: int, device="cpu"):
    """(cos_global, sin_global, cos_local, sin_local), each [max_pos, rot/2]."""
    from . import rope
    cg, sg = rope.build_tables(cfg, max_pos, device, theta=cfg.rope_theta)
    cl, sl = rope.build_tables(cfg, max_pos, device, theta=cfg.rope_local_theta or cfg.rope_theta)
    return cg, sg, cl, sl


@dataclass
class LaurelWeights:
    down: torch.Tensor   # [r, H]
    up: torch.Tensor     # [H, r]
    norm: torch.Tensor   # [H]


def laurel(x: torch.Tensor, attn_out: torch.Tensor, w: LaurelWeights, eps: float = 1e-6) -> torch.Tensor:
    """Learned augmented residual: (attn_out + x + norm(up(down(x)))) / sqrt(2)."""
    low = (x.float() @ w.down.float().t()) @ w.up.float().t()
    low = low * torch.rsqrt(low.pow(2).mean(-1, keepdim=True) + eps) * w.norm.float()
    return ((attn_out.float() + x.float() + low) / math.sqrt(2.0)).to(x.dtype)


@dataclass
class AltUpWeights:
    router: torch.Tensor        # [n, H]   modality router
    predict: torch.Tensor       # [n*n, n]
    correct: torch.Tensor       # [n, n]
    router_norm: torch.Tensor   # [H]
    out_scale: torch.Tensor     # [H]


def _altup_modalities(x_active: torch.Tensor, w: AltUpWeights, eps: float) -> torch.Tensor:
    h = x_active.float()
    h = h * torch.rsqrt(h.pow(2).mean(-1, keepdim=True) + eps) * w.router_norm.float()
    return torch.tanh((h @ w.router.float().t()) / x_active.shape[-1])      # [T, n]


def altup_predict(streams: torch.Tensor, w: AltUpWeights, active: int = 0, eps: float = 1e-6) -> torch.Tensor:
    """streams [n, T, H] -> predictions [n, T, H]: every stream is predicted as a routed mix of all streams."""
    n = streams.shape[0]
    mod = _altup_modalities(streams[active], w, eps)                          # [T, n]
    coef = (mod @ w.predict.float().t()).reshape(-1, n, n)                    # [T, n, n]
    pred = torch.einsum("tij,jth->ith", coef, streams.float())
    return (pred + streams.float()).to(streams.dtype)


def altup_correct(pred: torch.Tensor, activated: torch.Tensor, w: AltUpWeights, active: int = 0, eps: float = 1e-6) -> torch.Tensor:
    """The layer ran on the active stream only; spread its innovation (activated - predicted) to all streams."""
    mod = _altup_modalities(activated, w, eps)
    innov = activated.float() - pred[active].float()                          # [T, H]
    coef = (mod @ w.correct.float().t()) + 1.0                                # [T, n]
    return (pred.float() + coef.t()[:, :, None] * innov[None]).to(pred.dtype)


def altup_inject(corrected: torch.Tensor, ple: Optional[torch.Tensor], w: AltUpWeights, active: int = 0) -> torch.Tensor:
    """Per-layer embedding injected into the non-active streams after scaling the active output."""
    out = corrected.clone()
    out[active] = (corrected[active].float() * w.out_scale.float()).to(corrected.dtype)
    if ple is not None:
        for i in range(corrected.shape[0]):
            if i != active:
                out[i] = (corrected[i].float() + ple.float()).to(corrected.dtype)
    return out


def ple_gather(table: torch.Tensor, token_ids: torch.Tensor, layer: int, num_layers: int, scale: Optional[float] = None) -> torch.Tensor:
    """Per-layer embeddings: table [vocab, num_layers * d] -> this layer's [T, d] slice (scaled by sqrt(d))."""
    d = table.shape[1] // num_layers
    e = table[token_ids.long(), layer * d:(layer + 1) * d].float()
    return e * (math.sqrt(d) if scale is None else scale)
