"""Quantised-checkpoint tensor groups in SafeTensors: detection, dequantisation and repacking.

Reference parity:
  * AWQ / GPTQ  ``qweight/scales/qzeros/g_idx`` -> 72-byte / 128-element blocks ``[scale f16|pad|zero f16|pad|
    16 x u32 nibbles]``, zero stored as (z+1) for GPTQ, ``g_idx`` reorder (src/loader/awq_gptq_pairing.rs:47-219)
  * MXFP4 (gpt-oss) ``<p>_blocks`` (u8 e2m1, low nibble = even index) + ``<p>_scales`` (e8m0) [+ ``_bias``] ->
    GGUF 17-byte blocks (src/loader/mxfp4_pairing.rs:1-256)
  * NVFP4 ``<p>.weight`` U8 [N,K/2] + ``<p>.weight_scale`` ue4m3 [N,K/16] + ``<p>.weight_scale_2`` f32 ->
    64-element / 36-byte blocks (src/loader/nvfp4_pairing.rs:1-138)
  * FP8 per-tensor scale (src/fp8.rs:8-136). Block-scaled FP8 (``weight_scale_inv``, 128x128 tiles) and MXFP8
    (e4m3 + ue8m0 per 32) do not exist in the reference; they are defined here for the DeepSeek-V3 and
    Qwen3-MoE shapes.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional

import numpy as np
import torch

from . import quant

_AWQ_ORDER = [0, 4, 1, 5, 2, 6, 3, 7]  # AutoAWQ interleaves nibbles inside each int32


@dataclass
class QuantGroup:
    kind: str          # awq | gptq | mxfp4 | nvfp4 | fp8 | fp8_block | mxfp8
    prefix: str
    members: Dict[str, str]  # role -> tensor name


def detect_groups(names) -> List[QuantGroup]:
    names = set(names)
    out = []
    for n in sorted(names):
        if n.endswith(".qweight"):
            p = n[:-len(".qweight")]
            if p + ".scales" in names and p + ".qzeros" in names:
                kind = "gptq" if p + ".g_idx" in names else "awq"
                mem = {"qweight": n, "scales": p + ".scales", "qzeros": p + ".qzeros"}
                if kind == "gptq":
                    mem["g_idx"] = p + ".g_idx"
                out.append(QuantGroup(kind, p, mem))
        elif n.endswith("_blocks") and n[:-len("_blocks")] + "_scales" in names:
            p = n[:-len("_blocks")]
            mem = {"blocks": n, "scales": p + "_scales"}
            if p + "_bias" in names:
                mem["bias"] = p + "_bias"
            out.append(QuantGroup("mxfp4", p, mem))
        elif n.endswith(".weight_scale_inv"):
            p = n[:-len(".weight_scale_inv")]
            out.append(QuantGroup("fp8_block", p, {"weight": p + ".weight", "scale_inv": n}))
        elif n.endswith(".weight_scale"):
            p = n[:-len(".weight_scale")]
            if p + ".weight" in names:
                mem = {"weight": p + ".weight", "scale": n}
                if p + ".weight_scale_2" in names:
                    mem["scale2"] = p + ".weight_scale_2"
                out.append(QuantGroup("nvfp4_or_fp8", p, mem))
    return out


# ------------------------------------------------------------------------------------------------
# AWQ / GPTQ (4-bit, group size g along the input dimension)
# ------------------------------------------------------------------------------------------------
def _unpack_int32_nibbles(t: torch.Tensor, order=None) -> torch.Tensor:
    """[..., n] int32 -> [..., n*8] uint8 nibbles (element i of a word = bits 4i..4i+3, then reordered)."""
    w = t.to(torch.int64) & 0xFFFFFFFF
    nib = torch.stack([(w >> (4 * i)) & 0xF for i in range(8)], -1)
    if order is not None:
        inv = [order.index(i) for i in range(8)]
        nib = nib[..., inv]
    return nib.reshape(*t.shape[:-1], t.shape[-1] * 8).to(torch.uint8)


def dequant_awq(qweight, scales, qzeros) -> torch.Tensor:
    """AutoAWQ GEMM layout: qweight [K, N/8] i32, scales [K/g, N] f16, qzeros [K/g, N/8] i32 -> W [N, K] fp32."""
    K = qweight.shape[0]
    q = _unpack_int32_nibbles(qweight, _AWQ_ORDER).float()          # [K, N]
    z = _unpack_int32_nibbles(qzeros, _AWQ_ORDER).float()           # [K/g, N]
    g = K // scales.shape[0]
    w = (q - z.repeat_interleave(g, 0)) * scales.float().repeat_interleave(g, 0)
    return w.t().contiguous()


def dequant_gptq(qweight, scales, qzeros, g_idx=None) -> torch.Tensor:
    """AutoGPTQ layout: qweight [K/8, N] i32 (8 consecutive K per word), scales [K/g, N], qzeros [K/g, N/8] i32
    storing (zero - 1), optional g_idx [K] mapping each input row to its group -> W [N, K] fp32."""
    N = qweight.shape[1]
    w = qweight.t().contiguous()                                      # [N, K/8]
    q = _unpack_int32_nibbles(w).float()                              # [N, K]
    K = q.shape[1]
    z = ((_unpack_int32_nibbles(qzeros).to(torch.int32) + 1) & 0xF).float()   # stored as (zero - 1) mod 16
    if g_idx is None:
        g = K // scales.shape[0]
        g_idx = torch.arange(K) // g
    gi = g_idx.long()
    zz = z[gi].t()                                                    # [N, K]
    ss = scales.float()[gi].t()
    return ((q - zz) * ss).contiguous()


def repack_int4_blocks(w_q: torch.Tensor, scales: torch.Tensor, zeros: torch.Tensor) -> bytes:
    """[N, K] uint8 nibbles + per-(row, 128-group) scale/zero -> 72-byte blocks (type ids 50 / 51)."""
    N, K = w_q.shape
    assert K % 128 == 0
    nb = N * K // 128
    out = np.zeros((nb, 72), np.uint8)
    out[:, 0:2] = scales.reshape(-1).to(torch.float16).numpy().view(np.uint8).reshape(-1, 2)
    out[:, 4:6] = zeros.reshape(-1).to(torch.float16).numpy().view(np.uint8).reshape(-1, 2)
    q = w_q.reshape(nb, 16, 8).to(torch.int64)
    words = sum(q[:, :, i] << (4 * i) for i in range(8))
    out[:, 8:] = words.numpy().astype("<u4").view(np.uint8).reshape(nb, 64)
    return out.tobytes()


# ------------------------------------------------------------------------------------------------
# MXFP4 (gpt-oss SafeTensors) and NVFP4
# ------------------------------------------------------------------------------------------------
_E2M1 = torch.tensor([0, 0.5, 1, 1.5, 2, 3, 4, 6, -0.0, -0.5, -1, -1.5, -2, -3, -4, -6])


def dequant_mxfp4_st(blocks: torch.Tensor, scales: torch.Tensor) -> torch.Tensor:
    """blocks [..., G, 16] u8 (low nibble = even index), scales [..., G] e8m0 -> [..., G*32] fp32."""
    lo, hi = (blocks & 0xF).long(), (blocks >> 4).long()
    vals = torch.stack([_E2M1[lo], _E2M1[hi]], -1).reshape(*blocks.shape[:-1], 32)
    s = quant.e8m0_decode(scales)[..., None]
    return (vals * s).reshape(*blocks.shape[:-2], -1)


def repack_mxfp4_to_gguf(blocks: torch.Tensor, scales: torch.Tensor) -> bytes:
    """SafeTensors nibble order (even/odd interleaved) -> GGUF order (elements j and j+16 share a byte)."""
    b = blocks.reshape(-1, 16)
    lo, hi = b & 0xF, b >> 4
    elems = torch.stack([lo, hi], -1).reshape(-1, 32)                # element order
    packed = elems[:, :16] | (elems[:, 16:] << 4)
    out = torch.cat([scales.reshape(-1, 1), packed], 1)
    return out.numpy().astype(np.uint8).tobytes()


def dequant_nvfp4(weight: torch.Tensor, scale: torch.Tensor, scale2: Optional[torch.Tensor]) -> torch.Tensor:
    """weight [N, K/2] u8 (low nibble = even index), scale [N, K/16] ue4m3, scale2 global f32 -> [N, K] fp32."""
    N = weight.shape[0]
    lo, hi = (weight & 0xF).long(), (weight >> 4).long()
    vals = torch.stack([_E2M1[lo], _E2M1[hi]], -1).reshape(N, -1)
    s = scale.view(torch.float8_e4m3fn).float().repeat_interleave(16, 1)
    g = 1.0 if scale2 is None else float(scale2.reshape(-1)[0])
    return vals * s * g


def repack_nvfp4_blocks(weight: torch.Tensor, scale: torch.Tensor) -> bytes:
    """-> 64-element / 36-byte blocks [4 scales | 32 nibble bytes] (type id 53); the global scale stays apart."""
    N, Kh = weight.shape
    K = Kh * 2
    assert K % 64 == 0
    w = weight.reshape(N, K // 64, 32)
    s = scale.view(torch.uint8).reshape(N, K // 64, 4)
    return torch.cat([s, w], -1).reshape(-1).numpy().astype(np.uint8).tobytes()


# ------------------------------------------------------------------------------------------------
# FP8
# ------------------------------------------------------------------------------------------------
def dequant_fp8(weight: torch.Tensor, scale: Optional[torch.Tensor]) -> torch.Tensor:
    w = weight.float()
    if scale is None:
        return w
    s = scale.float()
    return w * (s if s.numel() == 1 else s.reshape(-1, 1))


def dequant_fp8_block(weight: torch.Tensor, scale_inv: torch.Tensor, block: int = 128) -> torch.Tensor:
    """DeepSeek-V3 layout: weight [N,K] e4m3, scale_inv [ceil(N/128), ceil(K/128)] f32 (multiply to dequantise)."""
    N, K = weight.shape
    s = scale_inv.float().repeat_interleave(block, 0)[:N].repeat_interleave(block, 1)[:, :K]
    return weight.float() * s


def quantize_fp8_block(w: torch.Tensor, block: int = 128):
    N, K = w.shape
    nb, kb = (N + block - 1) // block, (K + block - 1) // block
    pad = torch.zeros(nb * block, kb * block)
    pad[:N, :K] = w.float()
    amax = pad.reshape(nb, block, kb, block).abs().amax((1, 3)).clamp_min(1e-12)
    scale_inv = amax / 448.0
    q = (pad.reshape(nb, block, kb, block) / scale_inv[:, None, :, None]).reshape(nb * block, kb * block)[:N, :K]
    return q.to(torch.float8_e4m3fn), scale_inv


def quantize_mxfp8(w: torch.Tensor):
    """e4m3 values + ue8m0 scale per 32 consecutive K elements: returns (q [N,K] e4m3, scales [N,K/32] u8)."""
    N, K = w.shape
    g = w.float().reshape(N, K // 32, 32)
    amax = g.abs().amax(-1).clamp_min(2.0 ** -127)
    e = torch.clamp(torch.ceil(torch.log2(amax / 448.0)), -127, 127)
    scale = torch.exp2(e)
    q = (g / scale[..., None]).reshape(N, K).to(torch.float8_e4m3fn)
    return q, (e + 127).to(torch.uint8)


def dequant_mxfp8(q: torch.Tensor, scales: torch.Tensor) -> torch.Tensor:
    N, K = q.shape
    return (q.float().reshape(N, K // 32, 32) * quant.e8m0_decode(scales)[..., None]).reshape(N, K)


def dequant_group(group: QuantGroup, get) -> torch.Tensor:
    """Dequantise one detected group to an fp32 [out, in] weight. ``get(name)`` returns the raw tensor."""
    m = group.members
    if group.kind == "awq":
        return dequant_awq(get(m["qweight"]), get(m["scales"]), get(m["qzeros"]))
    if group.kind == "gptq":
        return dequant_gptq(get(m["qweight"]), get(m["scales"]), get(m["qzeros"]), get(m["g_idx"]) if "g_idx" in m else None)
    if group.kind == "mxfp4":
        return dequant_mxfp4_st(get(m["blocks"]), get(m["scales"]))
    if group.kind == "fp8_block":
        return dequant_fp8_block(get(m["weight"]), get(m["scale_inv"]))
    if group.kind == "nvfp4_or_fp8":
        w = get(m["weight"])
        if w.dtype == torch.uint8:
            return dequant_nvfp4(w, get(m["scale"]), get(m["scale2"]) if "scale2" in m else None)
        return dequant_fp8(w, get(m["scale"]))
    raise ValueError(group.kind)
