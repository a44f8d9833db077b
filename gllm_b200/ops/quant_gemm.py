"""Weight-quantised linear layers: the canonical quantised weight form, packers from every checkpoint format, and
the GEMM that dequantises inside its main loop.

Canonical form (``QuantWeight``): codes uint8 [N, K*bits/8] (4-bit: low nibble = even k), scales bf16 [N, K/group],
optional offsets bf16 [N, K/group]; value = decode(code) * scale + offset, decode by mode:
``fp8`` e4m3, ``fp4`` e2m1, ``int4`` unsigned nibble, ``int8`` signed byte.

Sources: MXFP8 (e4m3 + ue8m0 per 32), DeepSeek block-fp8 (128x128 ``weight_scale_inv``), per-tensor fp8, NVFP4
(e2m1 + ue4m3 per 16 + global), MXFP4 (e2m1 + ue8m0 per 32), AWQ / GPTQ int4 groups, GGUF Q4_0 / Q8_0 / Q4_K / Q6_K
(other GGUF types are dequantised to bf16 at load). CUDA path: ``csrc/kernels/qgemm_sm100.cu``; CPU path: fp32
matmul against ``dequantize()``.

Reference parity: ``QuantGemm`` (src/arch/auto_graph_fragments/build_graph.inc.rs:116) with the block layouts of
src/loader/{awq_gptq_pairing,mxfp4_pairing,nvfp4_pairing}.rs and src/loader/gguf/types.rs:152-236.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import numpy as np
import torch

from . import _native as nv
from ._native import F, I, L, P

nv.register("gllm_qgemm", I, [P, L, P, L, I, I, P, P, I, L, P, L, I, I, I, P, I, F, F, P, L, I, P])

MODES = {"fp8": 0, "fp4": 1, "int4": 2, "int8": 3}
_E2M1 = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0])


@dataclass
class QuantWeight:
    mode: str
    group: int
    codes: torch.Tensor                 # uint8 [N, K*bits/8]
    scales: torch.Tensor                # bf16 [N, K/group]
    offsets: Optional[torch.Tensor]     # bf16 [N, K/group]
    n: int
    k: int
    offset_in_codes: bool = False       # True: value = (code + offset) * scale (integer zero points stay exact)

    @property
    def bits(self) -> int:
        return 8 if self.mode in ("fp8", "int8") else 4

    @property
    def shape(self):
        return (self.n, self.k)

    def nbytes(self) -> int:
        return self.codes.numel() + 2 * self.scales.numel() + (0 if self.offsets is None else 2 * self.offsets.numel())

    def to(self, device) -> "QuantWeight":
        mv = lambda t: None if t is None else t.to(device).contiguous()
        return QuantWeight(self.mode, self.group, mv(self.codes), mv(self.scales), mv(self.offsets), self.n, self.k,
                           self.offset_in_codes)

    def decode_codes(self) -> torch.Tensor:
        c = self.codes
        if self.mode == "fp8":
            return c.view(torch.float8_e4m3fn).float()
        if self.mode == "int8":
            return c.view(torch.int8).float()
        lo, hi = (c & 0xF).long(), (c >> 4).long()
        if self.mode == "fp4":
            tab = _E2M1.to(c.device)
            lo, hi = tab[lo], tab[hi]
        return torch.stack([lo.float(), hi.float()], -1).reshape(self.n, self.k)

    def dequantize(self, dtype=torch.float32) -> torch.Tensor:
        s = self.scales.float().repeat_interleave(self.group, 1)
        c = self.decode_codes()
        if self.offsets is None:
            return (c * s).to(dtype)
        o = self.offsets.float().repeat_interleave(self.group, 1)
        return ((c + o) * s if self.offset_in_codes else c * s + o).to(dtype)


def _bf16(x):
    return x.to(torch.bfloat16).contiguous()


def _pack_nibbles(q: torch.Tensor) -> torch.Tensor:
    """[N, K] codes < 16 -> [N, K/2] bytes, low nibble = even k."""
    q = q.to(torch.uint8)
    return (q[:, 0::2] | (q[:, 1::2] << 4)).contiguous()


# ------------------------------------------------------------------------------------------------
# from checkpoint formats
# ------------------------------------------------------------------------------------------------
def from_mxfp8(q: torch.Tensor, e8m0: torch.Tensor) -> QuantWeight:
    N, K = q.shape
    s = torch.exp2(e8m0.float() - 127.0)
    return QuantWeight("fp8", 32, q.view(torch.uint8).contiguous(), _bf16(s), None, N, K)


def from_fp8_block(q: torch.Tensor, scale_inv: torch.Tensor, block: int = 128) -> QuantWeight:
    """DeepSeek-V3 128x128 block scales -> one scale per (row, 128 k)."""
    N, K = q.shape
    s = scale_inv.float().repeat_interleave(block, 0)[:N]               # [N, ceil(K/128)]
    if K % block:
        raise ValueError("block-fp8: K must be a multiple of the block")
    return QuantWeight("fp8", block, q.view(torch.uint8).contiguous(), _bf16(s), None, N, K)


def from_fp8_tensor(q: torch.Tensor, scale) -> QuantWeight:
    N, K = q.shape
    g = 128
    while K % g:
        g //= 2
    s = torch.as_tensor(scale, dtype=torch.float32).reshape(-1)
    s = s.expand(N) if s.numel() == 1 else s
    return QuantWeight("fp8", g, q.view(torch.uint8).contiguous(), _bf16(s[:, None].expand(N, K // g)), None, N, K)


def from_nvfp4(weight: torch.Tensor, scale_ue4m3: torch.Tensor, scale2=None) -> QuantWeight:
    N, Kh = weight.shape
    s = scale_ue4m3.view(torch.float8_e4m3fn).float() * (1.0 if scale2 is None else float(torch.as_tensor(scale2).reshape(-1)[0]))
    return QuantWeight("fp4", 16, weight.contiguous(), _bf16(s), None, N, Kh * 2)


def from_mxfp4(blocks: torch.Tensor, e8m0: torch.Tensor) -> QuantWeight:
    """blocks [N, G, 16] u8 (low nibble = even index), scales [N, G] e8m0."""
    N, G, _ = blocks.shape
    return QuantWeight("fp4", 32, blocks.reshape(N, G * 16).contiguous(), _bf16(torch.exp2(e8m0.float() - 127.0)), None, N, G * 32)


def from_int4_groups(q: torch.Tensor, scales: torch.Tensor, zeros: torch.Tensor) -> QuantWeight:
    """q [N, K] codes 0..15, scales / zeros [N, K/g]: w = (q - z) * s."""
    N, K = q.shape
    g = K // scales.shape[1]
    return QuantWeight("int4", g, _pack_nibbles(q), _bf16(scales.float()), _bf16(-zeros.float()), N, K, offset_in_codes=True)


def from_awq(qweight, scales, qzeros) -> QuantWeight:
    from ..loader.pairing import _AWQ_ORDER, _unpack_int32_nibbles
    q = _unpack_int32_nibbles(qweight, _AWQ_ORDER).t().contiguous()            # [N, K]
    z = _unpack_int32_nibbles(qzeros, _AWQ_ORDER).t().contiguous()             # [N, K/g]
    return from_int4_groups(q, scales.t().contiguous(), z)


def from_gptq(qweight, scales, qzeros, g_idx=None) -> Optional[QuantWeight]:
    """None when ``g_idx`` is an activation-order permutation (groups not contiguous in k): caller dequantises."""
    from ..loader.pairing import _unpack_int32_nibbles
    q = _unpack_int32_nibbles(qweight.t().contiguous())                         # [N, K]
    K = q.shape[1]
    g = K // scales.shape[0]
    if g_idx is not None and not torch.equal(g_idx.long(), torch.arange(K) // g):
        return None
    z = ((_unpack_int32_nibbles(qzeros).to(torch.int32) + 1) & 0xF).t().contiguous()
    return from_int4_groups(q, scales.t().contiguous(), z)


def from_gguf(type_id: int, raw, n: int, k: int) -> Optional[QuantWeight]:
    """Exact repack of GGUF block formats that are affine per sub-block. Returns None for the others."""
    from ..loader.quant import BY_NAME

    class QT:
        Q8_0, Q4_0, Q4_K, Q6_K = (BY_NAME[x].id for x in ("Q8_0", "Q4_0", "Q4_K", "Q6_K"))
    b = np.frombuffer(raw, dtype=np.uint8)
    f16 = lambda a: torch.from_numpy(a.copy().view(np.float16).astype(np.float32))
    if type_id == QT.Q8_0:                    # 34 bytes: d f16, 32 x i8
        blk = b.reshape(n, k // 32, 34)
        d = f16(blk[:, :, :2]).reshape(n, k // 32)
        codes = torch.from_numpy(blk[:, :, 2:].copy()).reshape(n, k)
        return QuantWeight("int8", 32, codes.contiguous(), _bf16(d), None, n, k)
    if type_id == QT.Q4_0:                    # 18 bytes: d f16, 16 bytes (element j and j+16 share a byte), w = d * (q - 8)
        blk = b.reshape(n, k // 32, 18)
        d = f16(blk[:, :, :2]).reshape(n, k // 32)
        qs = torch.from_numpy(blk[:, :, 2:].copy())
        q = torch.cat([qs & 0xF, qs >> 4], -1).reshape(n, k)
        return QuantWeight("int4", 32, _pack_nibbles(q), _bf16(d), _bf16(torch.full_like(d, -8.0)), n, k, offset_in_codes=True)
    if type_id == QT.Q4_K:                    # 144 bytes per 256: d, dmin f16; 12 bytes 6-bit scales/mins; 128 bytes nibbles
        blk = b.reshape(n, k // 256, 144)
        d, dmin = f16(blk[:, :, 0:2]).reshape(n, -1), f16(blk[:, :, 2:4]).reshape(n, -1)
        sc = torch.from_numpy(blk[:, :, 4:16].copy()).long()
        ls, lm = torch.zeros(n, k // 256, 8), torch.zeros(n, k // 256, 8)
        for j in range(8):
            if j < 4:
                ls[..., j], lm[..., j] = sc[..., j] & 63, sc[..., j + 4] & 63
            else:
                ls[..., j] = (sc[..., j + 4] & 0xF) | ((sc[..., j - 4] >> 6) << 4)
                lm[..., j] = (sc[..., j + 4] >> 4) | ((sc[..., j] >> 6) << 4)
        qs = torch.from_numpy(blk[:, :, 16:].copy()).reshape(n, k // 256, 4, 32)
        q = torch.stack([qs & 0xF, qs >> 4], 3).reshape(n, k)                   # sub-blocks 2g (low) and 2g+1 (high)
        s = (d[..., None] * ls).reshape(n, k // 32)
        o = (-dmin[..., None] * lm).reshape(n, k // 32)
        return QuantWeight("int4", 32, _pack_nibbles(q), _bf16(s), _bf16(o), n, k)
    if type_id == QT.Q6_K:                    # 210 bytes per 256: ql 128, qh 64, scales i8 x16, d f16; w = d * sc * (q - 32)
        blk = b.reshape(n, k // 256, 210)
        ql = torch.from_numpy(blk[:, :, :128].copy()).long().reshape(n, -1, 2, 64)
        qh = torch.from_numpy(blk[:, :, 128:192].copy()).long().reshape(n, -1, 2, 32)
        sc = torch.from_numpy(blk[:, :, 192:208].copy().view(np.int8)).float()
        d = f16(blk[:, :, 208:210]).reshape(n, -1)
        parts = []
        for half in range(2):
            l, h = ql[:, :, half], qh[:, :, half]
            q1 = (l[..., :32] & 0xF) | (((h >> 0) & 3) << 4)
            q2 = (l[..., 32:] & 0xF) | (((h >> 2) & 3) << 4)
            q3 = (l[..., :32] >> 4) | (((h >> 4) & 3) << 4)
            q4 = (l[..., 32:] >> 4) | (((h >> 6) & 3) << 4)
            parts.append(torch.cat([q1, q2, q3, q4], -1))
        q = (torch.cat(parts, -1) - 32).reshape(n, k)
        s = (d[..., None] * sc).reshape(n, k // 16)
        return QuantWeight("int8", 16, q.to(torch.int8).view(torch.uint8).contiguous(), _bf16(s), None, n, k)
    return None


# ------------------------------------------------------------------------------------------------
# quantisers (load-time quantisation of a dense model, and test vectors)
# ------------------------------------------------------------------------------------------------
def quantize(w: torch.Tensor, mode: str = "fp8", group: int = 32) -> QuantWeight:
    N, K = w.shape
    g = w.float().reshape(N, K // group, group)
    if mode == "fp8":
        s = (g.abs().amax(-1) / 448.0).clamp_min(1e-12).to(torch.bfloat16).float()
        q = (g / s[..., None]).reshape(N, K).to(torch.float8_e4m3fn)
        return QuantWeight("fp8", group, q.view(torch.uint8).contiguous(), _bf16(s), None, N, K)
    if mode == "int8":
        s = (g.abs().amax(-1) / 127.0).clamp_min(1e-12).to(torch.bfloat16).float()
        q = torch.round(g / s[..., None]).clamp(-127, 127).reshape(N, K).to(torch.int8)
        return QuantWeight("int8", group, q.view(torch.uint8).contiguous(), _bf16(s), None, N, K)
    if mode == "int4":
        lo, hi = g.amin(-1), g.amax(-1)
        s = ((hi - lo) / 15.0).clamp_min(1e-12).to(torch.bfloat16).float()
        o = lo.to(torch.bfloat16).float()
        q = torch.round((g - o[..., None]) / s[..., None]).clamp(0, 15).reshape(N, K)
        return QuantWeight("int4", group, _pack_nibbles(q), _bf16(s), _bf16(o), N, K)
    if mode == "fp4":
        s = (g.abs().amax(-1) / 6.0).clamp_min(1e-12).to(torch.bfloat16).float()
        x = (g / s[..., None]).reshape(N, K)
        mag = _E2M1[:8]
        idx = (x.abs()[..., None] - mag).abs().argmin(-1)
        q = idx + (x < 0).long() * 8
        return QuantWeight("fp4", group, _pack_nibbles(q), _bf16(s), None, N, K)
    raise ValueError(mode)


# ------------------------------------------------------------------------------------------------
# the op
# ------------------------------------------------------------------------------------------------
_partial = {}


def _partial_scratch(device, floats: int):
    key = (device.type, device.index)
    t = _partial.get(key)
    if t is None or t.numel() < floats:
        t = _partial[key] = torch.empty(max(floats, 8 << 20), dtype=torch.float32, device=device)
    return t


def qgemm(a: torch.Tensor, qw: QuantWeight, *, out: Optional[torch.Tensor] = None, row_ss=None, norm_dim: int = 0,
          eps: float = 0.0, splits: int = 0) -> torch.Tensor:
    """out[M, N] = rowscale(a) @ dequant(qw)^T. ``row_ss`` (sum of squares per row) turns on the RMSNorm row scale
    (the norm weight must already be folded into ``qw`` before quantisation)."""
    M, K = a.shape
    if K != qw.k:
        raise ValueError(f"qgemm: a has K={K}, weight has K={qw.k}")
    if not a.is_cuda:
        x = a.float()
        if row_ss is not None:
            ss = row_ss.float().reshape(M, -1).sum(-1, keepdim=True)
            x = x * torch.rsqrt(ss / norm_dim + eps)
        y = (x @ qw.dequantize().t()).to(a.dtype)
        if out is not None:
            out.copy_(y)
            return out
        return y
    if a.dtype != torch.bfloat16:
        raise TypeError("qgemm needs bf16 activations on the GPU")
    if qw.codes.device != a.device:
        raise ValueError("quantised weight lives on another device: call .to(device) at load time")
    if out is None:
        out = torch.empty((M, qw.n), dtype=torch.bfloat16, device=a.device)
    parts = 0 if row_ss is None else (row_ss.shape[1] if row_ss.dim() > 1 else 1)
    scratch = _partial_scratch(a.device, 16 * M * out.stride(0))
    rc = nv.lib().gllm_qgemm(a.data_ptr(), a.stride(0), qw.codes.data_ptr(), qw.codes.stride(0), MODES[qw.mode], qw.group,
                             qw.scales.data_ptr(), nv.ptr(qw.offsets), 1 if qw.offset_in_codes else 0, qw.scales.stride(0),
                             out.data_ptr(), out.stride(0),
                             M, qw.n, K, nv.ptr(row_ss), parts, 1.0 / norm_dim if norm_dim else 0.0, float(eps),
                             scratch.data_ptr(), scratch.numel(), int(splits), nv.stream_ptr())
    nv.check(rc, "qgemm")
    return out
