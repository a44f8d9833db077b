"""Quantised block formats: type table, CPU dequantisation (C++ ``libgllm_loader``), scalar codecs and the
reference quantisers used to build test checkpoints.

Reference parity: ``GgmlDType`` with 36 dtypes incl. custom ids 50-53 (src/loader/gguf/types.rs:57-94), block
sizes (:152-236), ``CpuBackend::dequantize`` dispatch (src/compat/cpu_backend.rs:1051-1159), FP8/FP4 scalar
codecs (src/fp8.rs:8-136, src/compat/weight_helpers.rs:501-870). Unlike the reference's truncating FP8
encoders, the encoders here round to nearest even and follow the OCP encodings (no infinities in e4m3).
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Dict

import numpy as np
import torch

from .._lib_loader import shared_lib_path


@dataclass(frozen=True)
class QuantType:
    id: int
    name: str
    block_elems: int
    block_bytes: int
    supported: bool = True


_T = [
    QuantType(0, "F32", 1, 4), QuantType(1, "F16", 1, 2), QuantType(2, "Q4_0", 32, 18), QuantType(3, "Q4_1", 32, 20),
    QuantType(6, "Q5_0", 32, 22), QuantType(7, "Q5_1", 32, 24), QuantType(8, "Q8_0", 32, 34),
    QuantType(9, "Q8_1", 32, 36), QuantType(10, "Q2_K", 256, 84), QuantType(11, "Q3_K", 256, 110),
    QuantType(12, "Q4_K", 256, 144), QuantType(13, "Q5_K", 256, 176), QuantType(14, "Q6_K", 256, 210),
    QuantType(15, "Q8_K", 256, 292),
    # codebook formats (lattice grids): decoded through the ``gguf`` package's tables when that package is importable
    # (it ships the grids of every IQ type), metadata only otherwise
    QuantType(16, "IQ2_XXS", 256, 66, False), QuantType(17, "IQ2_XS", 256, 74, False),
    QuantType(18, "IQ3_XXS", 256, 98, False), QuantType(19, "IQ1_S", 256, 50, False),
    QuantType(20, "IQ4_NL", 32, 18), QuantType(21, "IQ3_S", 256, 110, False), QuantType(22, "IQ2_S", 256, 82, False),
    QuantType(23, "IQ4_XS", 256, 136), QuantType(24, "I8", 1, 1), QuantType(25, "I16", 1, 2),
    QuantType(26, "I32", 1, 4), QuantType(27, "I64", 1, 8), QuantType(28, "F64", 1, 8),
    QuantType(29, "IQ1_M", 256, 56, False), QuantType(30, "BF16", 1, 2), QuantType(34, "TQ1_0", 256, 54),
    QuantType(35, "TQ2_0", 256, 66), QuantType(39, "MXFP4", 32, 17),
    QuantType(50, "AWQ4", 128, 72), QuantType(51, "GPTQ4", 128, 72), QuantType(52, "SQUEEZE", 128, 72, False),
    QuantType(53, "NVFP4", 64, 36),
]
TYPES: Dict[int, QuantType] = {t.id: t for t in _T}
BY_NAME: Dict[str, QuantType] = {t.name: t for t in _T}

_lib = None


def _native():
    global _lib
    if _lib is None:
        lib = ctypes.CDLL(str(shared_lib_path("libgllm_loader", "loader")))
        lib.gllm_dequantize.restype = ctypes.c_int
        lib.gllm_dequantize.argtypes = [ctypes.c_int, ctypes.c_void_p, ctypes.c_longlong, ctypes.c_void_p]
        lib.gllm_quant_block_info.restype = ctypes.c_int
        lib.gllm_quant_block_info.argtypes = [ctypes.c_int, ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_int)]
        _lib = lib
    return _lib


def nbytes(type_id: int, n_elems: int) -> int:
    t = TYPES[type_id]
    if n_elems % t.block_elems:
        raise ValueError(f"{n_elems} elements is not a multiple of the {t.name} block ({t.block_elems})")
    return n_elems // t.block_elems * t.block_bytes


def dequantize(type_id: int, raw, n_elems: int) -> torch.Tensor:
    """raw: bytes-like / uint8 array holding whole blocks -> fp32 tensor [n_elems]."""
    t = TYPES.get(type_id)
    if t is None:
        raise ValueError(f"unknown quant type id {type_id}")
    if not t.supported:
        return _dequantize_codebook(t, raw, n_elems)
    if t.name in ("I8", "I16", "I32", "I64", "F64"):
        dt = {"I8": np.int8, "I16": np.int16, "I32": np.int32, "I64": np.int64, "F64": np.float64}[t.name]
        return torch.from_numpy(np.frombuffer(raw, dtype=dt, count=n_elems).astype(np.float32))
    buf = np.frombuffer(raw, dtype=np.uint8, count=nbytes(type_id, n_elems))
    out = np.empty(n_elems, dtype=np.float32)
    rc = _native().gllm_dequantize(type_id, buf.ctypes.data, n_elems, out.ctypes.data)
    if rc != 0:
        raise RuntimeError(f"dequantize({t.name}) failed")
    return torch.from_numpy(out)


def codebook_backend_available() -> bool:
    try:
        import gguf.quants  # noqa: F401
        return True
    except Exception:
        return False


def _dequantize_codebook(t: QuantType, raw, n_elems: int) -> torch.Tensor:
    """IQ1 / IQ2 / IQ3 blocks index lattice codebooks of a few thousand entries. Those tables are data of the GGML
    format, not of this engine: when the ``gguf`` package (the format's own Python library) is installed its tables
    decode the blocks; without it the type stays metadata-only and the loader says so."""
    try:
        import gguf
        from gguf import quants as gq
    except Exception as exc:
        raise NotImplementedError(
            f"{t.name} needs the codebook grids of the GGML format; install the `gguf` package or convert the checkpoint") from exc
    qt = getattr(gguf.GGMLQuantizationType, t.name, None)
    if qt is None:
        raise NotImplementedError(f"the installed gguf package does not know {t.name}")
    n_bytes = nbytes(t.id, n_elems)
    buf = np.frombuffer(raw, dtype=np.uint8, count=n_bytes).reshape(n_elems // t.block_elems, t.block_bytes)
    out = gq.dequantize(buf, qt)
    return torch.from_numpy(np.ascontiguousarray(out, dtype=np.float32).reshape(-1))


# ------------------------------------------------------------------------------------------------
# reference quantisers (numpy) — used to write test checkpoints and by the .gllm converter
# ------------------------------------------------------------------------------------------------
def quantize_q8_0(x: np.ndarray) -> bytes:
    x = x.astype(np.float32).reshape(-1, 32)
    d = np.abs(x).max(1) / 127.0
    inv = np.where(d > 0, 1.0 / np.where(d > 0, d, 1), 0)
    q = np.clip(np.rint(x * inv[:, None]), -127, 127).astype(np.int8)
    out = np.zeros((x.shape[0], 34), np.uint8)
    out[:, :2] = d.astype(np.float16).view(np.uint8).reshape(-1, 2)
    out[:, 2:] = q.view(np.uint8)
    return out.tobytes()


def quantize_q4_0(x: np.ndarray) -> bytes:
    x = x.astype(np.float32).reshape(-1, 32)
    idx = np.abs(x).argmax(1)
    mx = x[np.arange(x.shape[0]), idx]
    d = mx / -8.0
    inv = np.where(d != 0, 1.0 / np.where(d != 0, d, 1), 0)
    q = np.clip(np.floor(x * inv[:, None] + 8.5), 0, 15).astype(np.uint8)
    out = np.zeros((x.shape[0], 18), np.uint8)
    out[:, :2] = d.astype(np.float16).view(np.uint8).reshape(-1, 2)
    out[:, 2:] = q[:, :16] | (q[:, 16:] << 4)
    return out.tobytes()


def quantize_q4_k(x: np.ndarray) -> bytes:
    """Simple (non-iterative) Q4_K encoder: per 32-element sub-block scale/min, 6-bit quantised."""
    x = x.astype(np.float32).reshape(-1, 8, 32)
    nb = x.shape[0]
    mn = np.minimum(x.min(2), 0)
    sc = (x.max(2) - mn) / 15.0
    d = sc.max(1) / 63.0
    dmin = (-mn).max(1) / 63.0
    d16, dmin16 = d.astype(np.float16), dmin.astype(np.float16)
    df, dminf = d16.astype(np.float32), dmin16.astype(np.float32)
    ls = np.where(df[:, None] > 0, np.clip(np.rint(sc / np.where(df[:, None] > 0, df[:, None], 1)), 0, 63), 0).astype(np.uint8)
    lm = np.where(dminf[:, None] > 0, np.clip(np.rint(-mn / np.where(dminf[:, None] > 0, dminf[:, None], 1)), 0, 63), 0).astype(np.uint8)
    eff_d = df[:, None] * ls
    eff_m = dminf[:, None] * lm
    q = np.where(eff_d[:, :, None] > 0, np.clip(np.rint((x + eff_m[:, :, None]) / np.where(eff_d[:, :, None] > 0, eff_d[:, :, None], 1)), 0, 15), 0).astype(np.uint8)
    out = np.zeros((nb, 144), np.uint8)
    out[:, 0:2] = d16.view(np.uint8).reshape(-1, 2)
    out[:, 2:4] = dmin16.view(np.uint8).reshape(-1, 2)
    scales = np.zeros((nb, 12), np.uint8)
    for j in range(8):
        if j < 4:
            scales[:, j] |= ls[:, j]
            scales[:, j + 4] |= lm[:, j]
        else:
            scales[:, j + 4] |= (ls[:, j] & 0xF) | ((lm[:, j] & 0xF) << 4)
            scales[:, j - 4] |= (ls[:, j] >> 4) << 6
            scales[:, j] |= (lm[:, j] >> 4) << 6
    out[:, 4:16] = scales
    qs = np.zeros((nb, 128), np.uint8)
    for g in range(4):
        qs[:, g * 32:(g + 1) * 32] = q[:, 2 * g] | (q[:, 2 * g + 1] << 4)
    out[:, 16:] = qs
    return out.tobytes()


def quantize_q6_k(x: np.ndarray) -> bytes:
    x = x.astype(np.float32).reshape(-1, 16, 16)
    nb = x.shape[0]
    amax_idx = np.abs(x).argmax(2)
    mx = np.take_along_axis(x, amax_idx[:, :, None], 2)[:, :, 0]
    sub = mx / -32.0
    big = np.abs(sub).argmax(1)
    d = sub[np.arange(nb), big] / -128.0
    d16 = d.astype(np.float16)
    df = d16.astype(np.float32)
    sc = np.where(df[:, None] != 0, np.clip(np.rint(sub / np.where(df[:, None] != 0, df[:, None], 1)), -128, 127), 0).astype(np.int8)
    eff = df[:, None] * sc
    q = np.where(eff[:, :, None] != 0, np.clip(np.rint(x / np.where(eff[:, :, None] != 0, eff[:, :, None], 1)), -32, 31), 0).astype(np.int8) + 32
    q = q.astype(np.uint8).reshape(nb, 256)
    out = np.zeros((nb, 210), np.uint8)
    ql = np.zeros((nb, 128), np.uint8)
    qh = np.zeros((nb, 64), np.uint8)
    for half in range(2):
        base = half * 128
        for l in range(32):
            q1, q2, q3, q4 = q[:, base + l], q[:, base + l + 32], q[:, base + l + 64], q[:, base + l + 96]
            ql[:, half * 64 + l] = (q1 & 0xF) | ((q3 & 0xF) << 4)
            ql[:, half * 64 + l + 32] = (q2 & 0xF) | ((q4 & 0xF) << 4)
            qh[:, half * 32 + l] = (q1 >> 4) | ((q2 >> 4) << 2) | ((q3 >> 4) << 4) | ((q4 >> 4) << 6)
    out[:, :128] = ql
    out[:, 128:192] = qh
    out[:, 192:208] = sc.view(np.uint8)
    out[:, 208:210] = d16.view(np.uint8).reshape(-1, 2)
    return out.tobytes()


_E2M1 = np.array([0, 0.5, 1, 1.5, 2, 3, 4, 6], np.float32)


def encode_e2m1(x: np.ndarray) -> np.ndarray:
    """fp32 -> 4-bit e2m1 codes (sign in bit 3), nearest value, ties to even code."""
    mag = np.abs(x)[..., None]
    code = np.abs(mag - _E2M1).argmin(-1).astype(np.uint8)
    return code | ((x < 0).astype(np.uint8) << 3)


def quantize_mxfp4(x: np.ndarray) -> bytes:
    x = x.astype(np.float32).reshape(-1, 32)
    amax = np.abs(x).max(1)
    e = np.where(amax > 0, np.floor(np.log2(np.where(amax > 0, amax, 1))) - 2, -127)
    e8 = np.clip(e + 127, 0, 254).astype(np.uint8)
    scale = np.ldexp(1.0, e8.astype(np.int32) - 127).astype(np.float32)
    codes = encode_e2m1(x / scale[:, None])
    out = np.zeros((x.shape[0], 17), np.uint8)
    out[:, 0] = e8
    out[:, 1:] = codes[:, :16] | (codes[:, 16:] << 4)
    return out.tobytes()


def encode_ue4m3(x: np.ndarray) -> np.ndarray:
    """positive fp32 -> unsigned e4m3 byte (round to nearest even, saturate at 448)."""
    t = torch.from_numpy(np.clip(x, 0, 448).astype(np.float32)).to(torch.float8_e4m3fn)
    return t.view(torch.uint8).numpy()


def quantize_nvfp4_blocks(x: np.ndarray) -> bytes:
    """64-element blocks: 4 ue4m3 scales (per 16) + 32 nibble bytes, low nibble = even element."""
    x = x.astype(np.float32).reshape(-1, 4, 16)
    amax = np.abs(x).max(2)
    s8 = encode_ue4m3(amax / 6.0)
    sf = torch.from_numpy(s8.copy()).view(torch.float8_e4m3fn).float().numpy()
    codes = encode_e2m1(np.where(sf[:, :, None] > 0, x / np.where(sf[:, :, None] > 0, sf[:, :, None], 1), 0))
    codes = codes.reshape(-1, 64)
    out = np.zeros((x.shape[0], 36), np.uint8)
    out[:, :4] = s8
    out[:, 4:] = codes[:, 0::2] | (codes[:, 1::2] << 4)
    return out.tobytes()


QUANTIZERS = {"Q8_0": quantize_q8_0, "Q4_0": quantize_q4_0, "Q4_K": quantize_q4_k, "Q6_K": quantize_q6_k,
              "MXFP4": quantize_mxfp4, "NVFP4": quantize_nvfp4_blocks}


# ------------------------------------------------------------------------------------------------
# scalar codecs
# ------------------------------------------------------------------------------------------------
def fp8_e4m3_encode(x: torch.Tensor) -> torch.Tensor:
    return x.to(torch.float8_e4m3fn)


def fp8_e5m2_encode(x: torch.Tensor) -> torch.Tensor:
    return x.to(torch.float8_e5m2)


def e8m0_decode(e: torch.Tensor) -> torch.Tensor:
    """ue8m0 byte -> 2^(e-127) (255 = NaN)."""
    v = torch.ldexp(torch.ones_like(e, dtype=torch.float32), e.to(torch.int32) - 127)
    return torch.where(e == 255, torch.full_like(v, float("nan")), v)


def int4_dequant(q: torch.Tensor, scale: torch.Tensor, zero=None) -> torch.Tensor:
    """(q - zero) * scale (src/quantization.rs:6-60)."""
    z = 0 if zero is None else zero
    return (q.float() - z) * scale
