"""RoPE cos/sin tables, computed once on the host in float64 like the reference does
(src/engine/mega_kernel/executor_core.inc.rs:780-822): half-split ("NeoX") pairing (i, i+half),
freq_i = theta^(-2i/d), table layout [position][half]. Scaling families: linear, dynamic (NTK by
length), ntk, yarn, longrope, llama3 (src/model_config_fragments/types.inc.rs:285-322).
"""
from __future__ import annotations

import math

import torch

from .config import ModelConfig, RopeScaling


def _yarn_find_dim(num_rot, dim, base, max_pos):
    return (dim * math.log(max_pos / (num_rot * 2 * math.pi))) / (2 * math.log(base))


def inv_frequencies(rot_dim: int, theta: float, rs: RopeScaling, max_pos: int):
    """Returns (inv_freq float64 [rot_dim/2], attention_factor)."""
    half = rot_dim // 2
    idx = torch.arange(0, half, dtype=torch.float64)
    inv = 1.0 / (theta ** (2.0 * idx / rot_dim))
    attn = 1.0
    k = rs.kind
    if k in ("none", "", "default"):
        pass
    elif k == "linear":
        inv = inv / rs.factor
    elif k in ("dynamic", "ntk"):
        orig = rs.original_max_position or max_pos
        f = rs.factor if k == "ntk" else max(1.0, (rs.factor * max_pos / orig) - (rs.factor - 1.0))
        base = theta * (f ** (rot_dim / max(rot_dim - 2, 1)))
        inv = 1.0 / (base ** (2.0 * idx / rot_dim))
    elif k == "llama3":
        orig = rs.original_max_position or 8192
        low_wl, high_wl = orig / rs.low_freq_factor, orig / rs.high_freq_factor
        wl = 2 * math.pi / inv
        smooth = (orig / wl - rs.low_freq_factor) / (rs.high_freq_factor - rs.low_freq_factor)
        scaled = torch.where(wl > low_wl, inv / rs.factor, inv)
        mid = (1 - smooth) * inv / rs.factor + smooth * inv
        inv = torch.where((wl <= low_wl) & (wl >= high_wl), mid, scaled)
    elif k == "yarn":
        orig = rs.original_max_position or max_pos
        low = max(math.floor(_yarn_find_dim(rs.beta_fast, rot_dim, theta, orig)), 0)
        high = min(math.ceil(_yarn_find_dim(rs.beta_slow, rot_dim, theta, orig)), rot_dim - 1)
        ramp = torch.clamp((idx - low) / max(high - low, 1e-3), 0, 1)
        mask = 1.0 - ramp
        inv = (inv / rs.factor) * (1 - mask) + inv * mask
        if rs.attention_factor is not None:
            attn = float(rs.attention_factor)
        else:
            def ms(scale, m):
                return 1.0 if scale <= 1 else 0.1 * m * math.log(scale) + 1.0
            attn = ms(rs.factor, rs.mscale) / ms(rs.factor, rs.mscale_all_dim) if rs.mscale_all_dim else ms(rs.factor, 1.0)
    elif k == "longrope":
        orig = rs.original_max_position or max_pos
        factors = rs.long_factor if (max_pos > orig and rs.long_factor) else rs.short_factor
        if factors:
            inv = inv / torch.tensor(factors[:half], dtype=torch.float64)
        scale = max_pos / orig
        attn = float(rs.attention_factor) if rs.attention_factor is not None else (
            1.0 if scale <= 1 else math.sqrt(1 + math.log(scale) / math.log(orig)))
    else:
        raise ValueError(f"unknown rope scaling {k}")
    return inv, attn


def build_tables(cfg: ModelConfig, max_pos: int, device="cpu", theta=None):
    """cos, sin: float32 [max_pos, rotary_dim/2]; returns (None, None) for models without RoPE."""
    rot = cfg.rotary_dim
    if rot <= 0:
        return None, None
    inv, attn = inv_frequencies(rot, theta or cfg.rope_theta, cfg.rope_scaling, max_pos)
    ang = torch.arange(max_pos, dtype=torch.float64)[:, None] * inv[None, :]
    cos = (ang.cos() * attn).float().contiguous().to(device)
    sin = (ang.sin() * attn).float().contiguous().to(device)
    return cos, sin
