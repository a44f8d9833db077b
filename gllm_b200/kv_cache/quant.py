"""KV quantisers: KIVI (per-channel K, per-token V, asymmetric 2/4 bit), fast Walsh-Hadamard rotation,
stochastic rounding with an unbiased 1-bit residual, and per-page fp8.

Reference parity: src/kv_cache/quant.rs:35-700 (KIVI / FWHT / RaBitQ), host requantisation
src/scheduler/kv_optimizer.rs:446-830. Tensors may live on any device; everything is plain tensor math so the
same code requantises pages resident in HBM.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional

import torch


def fwht(x: torch.Tensor) -> torch.Tensor:
    """Orthonormal fast Walsh-Hadamard transform over the last dim (power of two). Self-inverse."""
    n = x.shape[-1]
    if n & (n - 1):
        raise ValueError("FWHT needs a power-of-two length")
    y = x.float().clone()
    h = 1
    shape = y.shape
    while h < n:
        y = y.reshape(*shape[:-1], n // (2 * h), 2, h)
        a, b = y[..., 0, :], y[..., 1, :]
        y = torch.stack([a + b, a - b], -2).reshape(shape)
        h *= 2
    return y / math.sqrt(n)


def stochastic_round(x: torch.Tensor, generator: Optional[torch.Generator] = None) -> torch.Tensor:
    """Unbiased rounding: E[round(x)] = x."""
    lo = torch.floor(x)
    u = torch.rand(x.shape, generator=generator, device=x.device)
    return lo + (u < (x - lo)).to(x.dtype)


@dataclass
class KiviPage:
    bits: int
    k_q: torch.Tensor       # uint8 codes [tokens, D] (unpacked: one code per byte for clarity of tests)
    k_scale: torch.Tensor   # [D] per channel
    k_zero: torch.Tensor    # [D]
    v_q: torch.Tensor       # uint8 codes [tokens, D]
    v_scale: torch.Tensor   # [tokens] per token
    v_zero: torch.Tensor    # [tokens]
    rotated: bool = False

    def packed_bytes(self) -> int:
        t, d = self.k_q.shape
        return 2 * (t * d * self.bits // 8) + (2 * d + 2 * t) * 2


def _asym(x, dim, bits, stochastic, gen):
    lo, hi = x.amin(dim, keepdim=True), x.amax(dim, keepdim=True)
    scale = ((hi - lo) / (2 ** bits - 1)).clamp_min(1e-8)
    q = (x - lo) / scale
    q = stochastic_round(q, gen) if stochastic else torch.round(q)
    return q.clamp_(0, 2 ** bits - 1).to(torch.uint8), scale.squeeze(dim), lo.squeeze(dim)


def kivi_quantize_k(k: torch.Tensor, bits: int = 4, stochastic: bool = False, gen=None):
    """k [tokens, D] -> codes + per-CHANNEL scale / zero (outlier channels keep their own range)."""
    return _asym(k.float(), 0, bits, stochastic, gen)


def kivi_quantize_v(v: torch.Tensor, bits: int = 4, stochastic: bool = False, gen=None):
    """v [tokens, D] -> codes + per-TOKEN scale / zero."""
    return _asym(v.float(), 1, bits, stochastic, gen)


def kivi_quantize_page(k, v, bits=4, rotate=False, stochastic=False, gen=None) -> KiviPage:
    if rotate:
        k, v = fwht(k), fwht(v)
    kq, ks, kz = kivi_quantize_k(k, bits, stochastic, gen)
    vq, vs, vz = kivi_quantize_v(v, bits, stochastic, gen)
    return KiviPage(bits, kq, ks, kz, vq, vs, vz, rotated=rotate)


def kivi_dequantize(p: KiviPage):
    k = p.k_q.float() * p.k_scale[None, :] + p.k_zero[None, :]
    v = p.v_q.float() * p.v_scale[:, None] + p.v_zero[:, None]
    if p.rotated:
        k, v = fwht(k), fwht(v)
    return k, v


def pack_codes(codes: torch.Tensor, bits: int) -> torch.Tensor:
    """Pack uint8 codes (< 2^bits) along the last dim, little end first."""
    per = 8 // bits
    c = codes.reshape(*codes.shape[:-1], -1, per).to(torch.int32)
    out = torch.zeros(c.shape[:-1], dtype=torch.int32, device=codes.device)
    for i in range(per):
        out |= c[..., i] << (bits * i)
    return out.to(torch.uint8)


def unpack_codes(packed: torch.Tensor, bits: int) -> torch.Tensor:
    per = 8 // bits
    p = packed.to(torch.int32)
    parts = [((p >> (bits * i)) & (2 ** bits - 1)) for i in range(per)]
    return torch.stack(parts, -1).reshape(*packed.shape[:-1], -1).to(torch.uint8)


def fp8_quantize_page(x: torch.Tensor):
    """Per-page (per-tensor) scaled e4m3 with round-to-nearest-even. Returns (fp8 tensor, scale)."""
    amax = x.abs().amax().float().clamp_min(1e-12)
    scale = amax / 448.0
    return (x.float() / scale).to(torch.float8_e4m3fn), scale


def fp8_dequantize_page(q: torch.Tensor, scale: torch.Tensor, dtype=torch.bfloat16):
    return (q.float() * scale).to(dtype)


def residual_sign_bits(x: torch.Tensor, recon: torch.Tensor):
    """1-bit residual track (sign + mean magnitude per row): the XNOR pool of the dual-track cache."""
    r = x.float() - recon.float()
    return (r >= 0), r.abs().mean(-1)


def apply_residual(recon: torch.Tensor, signs: torch.Tensor, mag: torch.Tensor):
    return recon.float() + (signs.float() * 2 - 1) * mag[..., None]
