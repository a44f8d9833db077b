"""Block-scaled operands for the tensor-core kinds with hardware scale factors (sm_100a):

    MXFP8   e4m3 codes, one ue8m0 (power-of-two) scale per 32 elements along K     tcgen05.mma.kind::mxf8f6f4.block_scale
    NVFP4   e2m1 codes (two per byte), one ue4m3 scale per 16 elements + one fp32   tcgen05.mma.kind::mxf4nvf4.block_scale
            scale for the whole tensor                                               (scale_vec::4X)

Both operands of such a GEMM are block-scaled: weights are packed once at load time (from an MXFP8 / NVFP4 / MXFP4 /
block-fp8 checkpoint, or by quantising bf16 weights), activations are quantised on the device right before the GEMM
(``quantize_act``; the RMSNorm of the fused layer stays a row scale in the GEMM epilogue, so the raw residual stream is
what gets quantised). The reference lowers these formats through its generic ``QuantGemm`` op
(src/arch/auto_graph_fragments/build_graph.inc.rs:116) after pairing the checkpoint tensors
(src/loader/nvfp4_pairing.rs:1-138, src/loader/mxfp4_pairing.rs:126-256); 128x128 block-scaled fp8 does not exist
there and is re-quantised to MXFP8 here (its scales are arbitrary fp32 numbers, the hardware's are powers of two).

Scale-factor memory layout (what the kernel's bulk copies and ``tcgen05.cp`` expect): the scale matrix [rows, cols]
(cols = K / 32 or K / 16) is cut into chunks of 128 rows x 4 columns = 512 bytes, chunk (rb, cb) at
``(rb * (cols / 4) + cb) * 512``; inside a chunk scale (r, j) sits at byte ``(r % 32) * 16 + (r // 32) * 4 + j``.
CPU tensors run an fp32 oracle over the same quantised operands.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Optional

import torch

from . import _native as nv

MXFP8, NVFP4 = 2, 3            # operand modes of the kernel (csrc/kernels/gemm_sm100.cu: OPM_MXFP8 / OPM_NVFP4)
_E2M1 = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0])
FMT_NAMES = {"mxfp8": MXFP8, "nvfp4": NVFP4}


# --------------------------------------------------------------------------------------------
# scale-factor layout
# --------------------------------------------------------------------------------------------
def sf_swizzle(sf: torch.Tensor) -> torch.Tensor:
    """uint8 scale matrix [rows, cols] -> 1-D uint8 in 512-byte chunks (rows padded to 128, cols to 4)."""
    assert sf.dtype == torch.uint8 and sf.dim() == 2
    R, C = sf.shape
    Rp, Cp = (R + 127) // 128 * 128, (C + 3) // 4 * 4
    if (Rp, Cp) != (R, C):
        pad = torch.zeros((Rp, Cp), dtype=torch.uint8, device=sf.device)
        pad[:R, :C] = sf
        sf = pad
    # [rb, r1 (4), r0 (32), cb, j (4)] -> [rb, cb, r0, r1, j]
    t = sf.view(Rp // 128, 4, 32, Cp // 4, 4).permute(0, 3, 2, 1, 4)
    return t.contiguous().view(-1)


def sf_unswizzle(buf: torch.Tensor, rows: int, cols: int) -> torch.Tensor:
    """The first ``rows`` rows of the scale matrix stored in ``buf`` (which may cover more row blocks than that)."""
    Rp, Cp = (rows + 127) // 128 * 128, (cols + 3) // 4 * 4
    need = (Rp // 128) * (Cp // 4) * 512
    t = buf[:need].view(Rp // 128, Cp // 4, 32, 4, 4).permute(0, 3, 2, 1, 4).contiguous().view(Rp, Cp)
    return t[:rows, :cols]


def sf_bytes(rows: int, cols: int) -> int:
    return ((rows + 127) // 128) * ((cols + 3) // 4) * 512


# --------------------------------------------------------------------------------------------
# codecs (fp32 host math; IEEE / OCP conformant roundings)
# --------------------------------------------------------------------------------------------
def ue8m0_encode(scale: torch.Tensor) -> torch.Tensor:
    """Power-of-two scales -> biased exponent bytes (value = 2 ** (byte - 127))."""
    e = torch.log2(scale.float().clamp_min(2.0 ** -127)).round().clamp(-127, 127)
    return (e + 127).to(torch.uint8)


def ue8m0_decode(b: torch.Tensor) -> torch.Tensor:
    return torch.exp2(b.float() - 127.0)


def e4m3_encode(x: torch.Tensor) -> torch.Tensor:
    return x.float().clamp(-448.0, 448.0).to(torch.float8_e4m3fn).view(torch.uint8)


def e4m3_decode(b: torch.Tensor) -> torch.Tensor:
    return b.view(torch.float8_e4m3fn).float()


def e2m1_encode(x: torch.Tensor) -> torch.Tensor:
    """fp32 -> 4-bit codes (sign bit 8), round to nearest, ties to the even code, saturating at 6."""
    a = x.float().abs().clamp(max=6.0)
    grid = _E2M1.to(x.device)
    mid = (grid[1:] + grid[:-1]) / 2
    idx = torch.bucketize(a, mid, right=False)            # a == midpoint -> lower code
    up = (a[..., None] == mid).any(-1) & (idx % 2 == 1)   # ... unless the lower code is odd: ties go to the even code
    idx = idx + up.to(idx.dtype)
    return (idx.to(torch.uint8) | ((x < 0).to(torch.uint8) << 3)).to(torch.uint8)


def e2m1_decode(c: torch.Tensor) -> torch.Tensor:
    v = _E2M1.to(c.device)[(c & 7).long()]
    return torch.where((c & 8) != 0, -v, v)


def pack_nibbles(c: torch.Tensor) -> torch.Tensor:
    """[.., K] codes -> [.., K/2] bytes, element 2i in the low nibble."""
    return (c[..., 0::2] | (c[..., 1::2] << 4)).contiguous()


def unpack_nibbles(b: torch.Tensor) -> torch.Tensor:
    out = torch.stack([b & 0xF, b >> 4], -1)
    return out.view(*b.shape[:-1], b.shape[-1] * 2)


# --------------------------------------------------------------------------------------------
# operands
# --------------------------------------------------------------------------------------------
@dataclass
class BlockScaled:
    """One block-scaled operand [rows, K]: codes, swizzled scale chunks, per-tensor scale."""
    fmt: int
    rows: int
    k: int
    codes: torch.Tensor         # uint8 [rows, K] (MXFP8) or [rows, K/2] (NVFP4)
    sf: torch.Tensor            # uint8, swizzled chunks
    tensor_scale: float = 1.0   # NVFP4 second-level scale (1.0 for MXFP8)

    @property
    def vec(self) -> int:
        return 32 if self.fmt == MXFP8 else 16

    @property
    def device(self):
        return self.codes.device

    def to(self, device) -> "BlockScaled":
        return BlockScaled(self.fmt, self.rows, self.k, self.codes.to(device), self.sf.to(device), self.tensor_scale)

    def nbytes(self) -> int:
        return self.codes.numel() + self.sf.numel()

    def scales(self) -> torch.Tensor:
        raw = sf_unswizzle(self.sf, self.rows, self.k // self.vec)
        return ue8m0_decode(raw) if self.fmt == MXFP8 else e4m3_decode(raw)

    def dequantize(self) -> torch.Tensor:
        """fp32 [rows, K]: exactly the values the tensor core multiplies (times tensor_scale)."""
        codes = self.codes[:self.rows]      # activation buffers are allocated for more rows than they hold
        if self.fmt == MXFP8:
            v = e4m3_decode(codes)
        else:
            v = e2m1_decode(unpack_nibbles(codes))
        s = self.scales().repeat_interleave(self.vec, dim=1)
        return v * s * self.tensor_scale


def _pad_k(x: torch.Tensor, mult: int) -> torch.Tensor:
    K = x.shape[1]
    if K % mult == 0:
        return x
    return torch.nn.functional.pad(x, (0, mult - K % mult))


def quantize_mxfp8(x: torch.Tensor) -> BlockScaled:
    """[rows, K] -> MXFP8 (K padded to 128 with zeros). Scale = smallest power of two with amax / scale <= 448."""
    x = _pad_k(x.float(), 128)
    R, K = x.shape
    blk = x.view(R, K // 32, 32)
    amax = blk.abs().amax(-1)
    e = torch.ceil(torch.log2((amax / 448.0).clamp_min(2.0 ** -127)))
    scale = torch.exp2(e)
    codes = e4m3_encode(blk / scale[..., None]).view(R, K)
    return BlockScaled(MXFP8, R, K, codes.contiguous(), sf_swizzle(ue8m0_encode(scale)), 1.0)


def quantize_nvfp4(x: torch.Tensor, tensor_scale: Optional[float] = None) -> BlockScaled:
    """[rows, K] -> NVFP4 (K padded to 256). tensor_scale defaults to amax / (6 * 448), the usual two-level recipe.
    The arithmetic (reciprocal multiplies in fp32, block scale rounded to ue4m3 before the codes are taken against it)
    is the device kernel's, operation for operation, so both produce the same bytes."""
    import numpy as np
    x = _pad_k(x.float(), 256)
    R, K = x.shape
    if tensor_scale is None:
        tensor_scale = max(float(x.abs().max()) / (6.0 * 448.0), 1e-12)
    inv_ts = float(np.float32(1.0) / np.float32(tensor_scale))
    sixth = float(np.float32(1.0) / np.float32(6.0))
    blk = x.view(R, K // 16, 16) * inv_ts
    s = e4m3_decode(e4m3_encode(blk.abs().amax(-1) * sixth))            # ue4m3: the positive half of e4m3
    inv = torch.where(s > 0, 1.0 / s, torch.zeros_like(s))
    codes = e2m1_encode(blk * inv[..., None]).view(R, K)
    return BlockScaled(NVFP4, R, K, pack_nibbles(codes), sf_swizzle(e4m3_encode(s)), float(np.float32(tensor_scale)))


def quantize(x: torch.Tensor, fmt) -> BlockScaled:
    fmt = FMT_NAMES.get(fmt, fmt)
    return quantize_mxfp8(x) if fmt == MXFP8 else quantize_nvfp4(x)


def from_mxfp8_checkpoint(q: torch.Tensor, e8m0: torch.Tensor) -> BlockScaled:
    """MXFP8 checkpoint tensors: e4m3 codes [N, K] and ue8m0 scales [N, K/32] (taken as they are)."""
    N, K = q.shape
    assert K % 128 == 0, "MXFP8 weights need K % 128 == 0"
    return BlockScaled(MXFP8, N, K, q.view(torch.uint8).contiguous(), sf_swizzle(e8m0.view(torch.uint8).contiguous()), 1.0)


def from_nvfp4_checkpoint(weight: torch.Tensor, scale_ue4m3: torch.Tensor, scale2=None) -> BlockScaled:
    """NVFP4 checkpoint tensors (HF layout): ``.weight`` u8 [N, K/2] (low nibble = even element), ``.weight_scale`` u8
    ue4m3 [N, K/16], ``.weight_scale_2`` fp32 (src/loader/nvfp4_pairing.rs:1-138)."""
    N, K2 = weight.shape
    assert (2 * K2) % 256 == 0, "NVFP4 weights need K % 256 == 0"
    ts = float(scale2) if scale2 is not None else 1.0
    return BlockScaled(NVFP4, N, 2 * K2, weight.view(torch.uint8).contiguous(),
                       sf_swizzle(scale_ue4m3.view(torch.uint8).contiguous()), ts)


def from_fp8_block_checkpoint(q: torch.Tensor, scale_inv: torch.Tensor, block: int = 128) -> BlockScaled:
    """128x128 block-scaled fp8 (DeepSeek-V3 style ``weight_scale_inv``): the scales are arbitrary fp32 numbers, the
    hardware's are powers of two, so the weight is re-quantised to MXFP8 (one more e4m3 rounding at load time)."""
    N, K = q.shape
    s = scale_inv.float().repeat_interleave(block, 0)[:N].repeat_interleave(block, 1)[:, :K]
    return quantize_mxfp8(q.view(torch.float8_e4m3fn).float() * s)


# --------------------------------------------------------------------------------------------
# device-side activation quantisation
# --------------------------------------------------------------------------------------------
nv.register("gllm_quantize_act", ctypes.c_int, [nv.P, nv.L, nv.I, nv.I, nv.I, nv.P, nv.L, nv.P, nv.F, nv.P])
nv.register("gllm_quantize_act_rows", ctypes.c_int, [nv.P, nv.L, nv.I, nv.I, nv.I, nv.P, nv.L, nv.P, nv.F, nv.P, nv.P])
nv.register("gllm_quantize_act_scatter", ctypes.c_int, [nv.P, nv.L, nv.I, nv.I, nv.I, nv.I, nv.P, nv.L, nv.P, nv.F, nv.P, nv.P])


def quantize_act(x: torch.Tensor, fmt, *, out: Optional[BlockScaled] = None, tensor_scale: float = 1.0) -> BlockScaled:
    """bf16 activations [M, K] -> block-scaled operand on the same device. ``tensor_scale`` (NVFP4 only) is a static
    second-level scale: values up to 6 * 448 * tensor_scale are representable."""
    fmt = FMT_NAMES.get(fmt, fmt)
    M, K = x.shape
    if not x.is_cuda:
        return quantize_mxfp8(x) if fmt == MXFP8 else quantize_nvfp4(x, tensor_scale)
    mult = 128 if fmt == MXFP8 else 256
    assert x.dtype == torch.bfloat16 and x.stride(1) == 1 and K % mult == 0, "activations: bf16, K % 128 (256 for NVFP4)"
    if out is None:
        out = alloc_act(M, K, fmt, x.device)
    out.rows, out.tensor_scale = M, (tensor_scale if fmt == NVFP4 else 1.0)
    rc = nv.lib().gllm_quantize_act(x.data_ptr(), x.stride(0), M, K, fmt, out.codes.data_ptr(), out.codes.stride(0),
                                    out.sf.data_ptr(), float(tensor_scale), nv.stream_ptr())
    nv.check(rc, "quantize_act")
    return out


def quantize_act_rows(x: torch.Tensor, fmt, out: BlockScaled, rows_limit: torch.Tensor, *, tensor_scale: float = 1.0):
    """Like ``quantize_act`` for the first ``rows_limit[0]`` rows of ``x`` (a count that lives on the device, e.g. the
    routed rows of an MoE step); the launch is sized for all of ``x``."""
    fmt = FMT_NAMES.get(fmt, fmt)
    M, K = x.shape
    if not x.is_cuda:
        n = int(rows_limit[0])
        q = quantize_mxfp8(x[:n]) if fmt == MXFP8 else quantize_nvfp4(x[:n], tensor_scale)
        return _host_update(out, q, torch.arange(n), M)
    out.rows, out.tensor_scale = M, (tensor_scale if fmt == NVFP4 else 1.0)
    rc = nv.lib().gllm_quantize_act_rows(x.data_ptr(), x.stride(0), M, K, fmt, out.codes.data_ptr(), out.codes.stride(0),
                                         out.sf.data_ptr(), float(tensor_scale), rows_limit.data_ptr(), nv.stream_ptr())
    nv.check(rc, "quantize_act_rows")
    return out


def quantize_act_scatter(x: torch.Tensor, dest: torch.Tensor, k: int, fmt, out: BlockScaled, rows: int, *,
                         tensor_scale: float = 1.0):
    """Routed MoE rows: pair (token t, slot j) = unit t * k + j reads row t of ``x`` and is written, quantised, to
    row ``dest[t * k + j]`` of ``out`` (negative: skipped). ``rows`` is the row count ``out`` then stands for."""
    fmt = FMT_NAMES.get(fmt, fmt)
    T, K = x.shape
    if not x.is_cuda:
        d = dest[:T * k].long()
        ok = d >= 0
        src = (torch.arange(T * k) // k)[ok]
        q = quantize_mxfp8(x[src]) if fmt == MXFP8 else quantize_nvfp4(x[src], tensor_scale)
        return _host_update(out, q, d[ok], rows)
    out.rows, out.tensor_scale = rows, (tensor_scale if fmt == NVFP4 else 1.0)
    rc = nv.lib().gllm_quantize_act_scatter(x.data_ptr(), x.stride(0), T * k, k, K, fmt, out.codes.data_ptr(),
                                            out.codes.stride(0), out.sf.data_ptr(), float(tensor_scale), dest.data_ptr(),
                                            nv.stream_ptr())
    nv.check(rc, "quantize_act_scatter")
    return out


def _host_update(out: BlockScaled, q: BlockScaled, rows_idx: torch.Tensor, rows: int) -> BlockScaled:
    """CPU oracle of the row-mapped quantisers: place the rows of ``q`` at ``rows_idx`` of ``out``."""
    cols = out.k // out.vec
    total = out.codes.shape[0]
    sf = sf_unswizzle(out.sf, total, cols).clone()
    if q.rows:
        out.codes[rows_idx] = q.codes
        sf[rows_idx] = sf_unswizzle(q.sf, q.rows, cols)
    out.sf = sf_swizzle(sf)
    out.rows, out.tensor_scale = rows, q.tensor_scale
    return out


def alloc_act(max_rows: int, K: int, fmt, device) -> BlockScaled:
    """Reusable output buffers of ``quantize_act`` for up to ``max_rows`` rows (rows padded to 256 for two-row tiles)."""
    fmt = FMT_NAMES.get(fmt, fmt)
    rows = (max_rows + 255) // 256 * 256
    kb = K if fmt == MXFP8 else K // 2
    codes = torch.zeros((rows, kb), dtype=torch.uint8, device=device)
    sf = torch.zeros(sf_bytes(rows, K // (32 if fmt == MXFP8 else 16)), dtype=torch.uint8, device=device)
    return BlockScaled(fmt, max_rows, K, codes, sf, 1.0)


# --------------------------------------------------------------------------------------------
# the GEMM
# --------------------------------------------------------------------------------------------
class _Args(ctypes.Structure):
    _fields_ = [("a", nv.P), ("lda", nv.L), ("sfa", nv.P), ("b", nv.P), ("ldb", nv.L), ("sfb", nv.P),
                ("out", nv.P), ("ldo", nv.L),
                ("M", nv.I), ("N", nv.I), ("K", nv.I), ("fmt", nv.I), ("epi", nv.I), ("out_f32", nv.I), ("bn", nv.I),
                ("max_ctas", nv.I), ("force_splits", nv.I), ("out_scale", nv.F), ("bias", nv.P),
                ("row_ss_in", nv.P), ("ss_in_parts", nv.I), ("norm_inv_dim", nv.F), ("norm_eps", nv.F),
                ("residual", nv.P), ("ldr", nv.L), ("row_ss_out", nv.P), ("glu_act", nv.I),
                ("mblk_group", nv.P), ("num_groups", nv.I),
                ("n_q_heads", nv.I), ("n_kv_heads", nv.I), ("q_out", nv.P), ("kv_cache", nv.P), ("num_pages", nv.I),
                ("slot_mapping", nv.P), ("positions", nv.P), ("cos_table", nv.P), ("sin_table", nv.P), ("max_pos", nv.I),
                ("q_norm_w", nv.P), ("k_norm_w", nv.P), ("qk_eps", nv.F), ("kv_inv_scale", nv.F), ("stream", nv.P),
                ("scatter_meta", nv.P), ("scatter_peer", nv.P), ("scatter_world", nv.I),
                ("ar_world", nv.I), ("ar_rank", nv.I), ("ar_mc_base", nv.P), ("ar_peer_base", nv.P),
                ("ar_region_bytes", nv.L), ("ar_recv_off", nv.L), ("ar_recv_bytes", nv.L), ("ar_res_off", nv.L),
                ("ar_res_bytes", nv.L), ("ar_state", nv.P)]


nv.register("gllm_gemm_blockscaled", ctypes.c_int, [ctypes.POINTER(_Args)])
EPI_STORE, EPI_RESIDUAL, EPI_GLU, EPI_QKV = 0, 1, 2, 3


def _base_args(a: BlockScaled, w: BlockScaled, M: int, N: int, epi: int, bn: int, splits: int, max_ctas: int) -> _Args:
    if a.fmt != w.fmt or a.k != w.k:
        raise ValueError(f"operand formats / K differ: {a.fmt}/{a.k} vs {w.fmt}/{w.k}")
    if a.device != w.device:
        raise ValueError(f"operands on {a.device} and {w.device}")
    g = _Args()
    g.a, g.lda, g.sfa = a.codes.data_ptr(), a.codes.stride(0), a.sf.data_ptr()
    g.b, g.ldb, g.sfb = w.codes.data_ptr(), w.codes.stride(0), w.sf.data_ptr()
    g.M, g.N, g.K, g.fmt, g.epi, g.bn = M, N, a.k, a.fmt, epi, bn
    g.max_ctas, g.force_splits = max_ctas, splits
    g.out_scale = float(a.tensor_scale * w.tensor_scale)
    g.stream = nv.stream_ptr()
    return g


def _ref_acc(a: BlockScaled, w: BlockScaled, M: int, row_ss=None, norm_dim=0, eps=0.0):
    from .linear import row_scale_ref
    acc = a.dequantize()[:M] @ w.dequantize().t()
    rs = row_scale_ref(row_ss, norm_dim, eps)
    return acc if rs is None else acc * rs[:M, None]


def gemm(a: BlockScaled, w: BlockScaled, *, out=None, out_dtype=torch.bfloat16, bias=None, row_ss=None, norm_dim=0,
         eps=0.0, bn: int = 128, splits: int = 0, max_ctas: int = 0, mblk_group=None, num_groups: int = 0):
    """out[M, N] = rowscale * (A @ W.T) (+ bias) with both operands block-scaled. With ``mblk_group`` W is a stack of
    ``num_groups`` [N, K] expert weights and 128-row block i of A multiplies expert ``mblk_group[i]`` (< 0: skipped)."""
    M = a.rows
    N = w.rows if mblk_group is None else w.rows // num_groups
    if not a.codes.is_cuda:
        if mblk_group is None:
            acc = _ref_acc(a, w, M, row_ss, norm_dim, eps)
        else:
            A, W = a.dequantize()[:M], w.dequantize()
            acc = torch.zeros((M, N))
            for i in range((M + 127) // 128):
                gi = int(mblk_group[i])
                if gi >= 0:
                    acc[i * 128:(i + 1) * 128] = A[i * 128:(i + 1) * 128] @ W[gi * N:(gi + 1) * N].t()
        if bias is not None:
            acc = acc + bias.float()
        res = acc.to(out.dtype if out is not None else out_dtype)
        if out is not None:
            out.copy_(res)
            return out
        return res
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=a.device)
    nv.ensure_splitk_workspace(a.device)
    g = _base_args(a, w, M, N, EPI_STORE, bn, 1 if mblk_group is not None else splits, max_ctas)
    g.out, g.ldo, g.out_f32 = out.data_ptr(), out.stride(0), 1 if out.dtype == torch.float32 else 0
    g.bias = nv.ptr(bias)
    if row_ss is not None:
        g.row_ss_in, g.ss_in_parts = row_ss.data_ptr(), (row_ss.shape[1] if row_ss.dim() > 1 else 1)
        g.norm_inv_dim, g.norm_eps = 1.0 / norm_dim, eps
    if mblk_group is not None:
        g.mblk_group, g.num_groups = mblk_group.data_ptr(), num_groups
    nv.check(nv.lib().gllm_gemm_blockscaled(ctypes.byref(g)), "gemm_blockscaled")
    return out


def gemm_grouped_scatter(a: BlockScaled, w: BlockScaled, mblk_group, num_groups: int, *, ldo: int, scatter_meta,
                         scatter_peers, world: int, bn: int = 128):
    """Grouped GEMM (row block i of A times expert ``mblk_group[i]``) whose output rows go straight into up to eight
    ranks' buffers: ``scatter_meta`` holds (rank, row) per input row, ``scatter_peers`` is a ctypes array of the
    ranks' base pointers, ``ldo`` the row pitch of those buffers in elements. CUDA only (the expert-parallel path)."""
    M = a.rows
    N = w.rows // num_groups
    nv.ensure_splitk_workspace(a.device)
    g = _base_args(a, w, M, N, EPI_STORE, bn, 1, 0)
    g.ldo = ldo
    g.mblk_group, g.num_groups = mblk_group.data_ptr(), num_groups
    g.scatter_meta, g.scatter_peer, g.scatter_world = scatter_meta.data_ptr(), ctypes.cast(scatter_peers, ctypes.c_void_p), world
    nv.check(nv.lib().gllm_gemm_blockscaled(ctypes.byref(g)), "gemm_blockscaled (scatter)")


def gemm_residual(a: BlockScaled, w: BlockScaled, residual, *, out=None, row_ss_out=None, bias=None, bn: int = 128,
                  splits: int = 0):
    """out = A @ W.T (+ bias) + residual (bf16); row_ss_out[M, ceil(N / bn)] = per-tile sums of squares of out."""
    M, N = a.rows, w.rows
    parts = (N + bn - 1) // bn
    if not a.codes.is_cuda:
        acc = _ref_acc(a, w, M)
        if bias is not None:
            acc = acc + bias.float()
        res = (acc + residual.float()).to(residual.dtype)
        ss = torch.nn.functional.pad(res.float().pow(2), (0, parts * bn - N)).reshape(M, parts, bn).sum(-1)
        if out is not None:
            out.copy_(res)
            res = out
        if row_ss_out is not None:
            row_ss_out[:M, :parts].copy_(ss)
            ss = row_ss_out
        return res, ss
    if out is None:
        out = torch.empty((M, N), dtype=torch.bfloat16, device=a.device)
    if row_ss_out is None:
        row_ss_out = torch.empty((M, parts), dtype=torch.float32, device=a.device)
    assert row_ss_out.shape[-1] == parts and row_ss_out.is_contiguous()
    nv.ensure_splitk_workspace(a.device)
    g = _base_args(a, w, M, N, EPI_RESIDUAL, bn, splits, 0)
    g.out, g.ldo, g.bias = out.data_ptr(), out.stride(0), nv.ptr(bias)
    g.residual, g.ldr, g.row_ss_out = residual.data_ptr(), residual.stride(0), row_ss_out.data_ptr()
    nv.check(nv.lib().gllm_gemm_blockscaled(ctypes.byref(g)), "gemm_blockscaled_residual")
    return out, row_ss_out


def gemm_residual_allreduce(a: BlockScaled, w: BlockScaled, x, row_ss_out, *, bn: int, world: int, rank: int, mc_base,
                            peer_base, region_bytes: int, recv_off: int, recv_bytes: int, res_off: int, res_bytes: int,
                            state):
    """x <- sum over ranks of (A @ W.T) + x in one kernel: the block-scaled row-parallel GEMM with the low-latency
    all-reduce of ``parallel.tensor_parallel.TPContext`` in its epilogue (partials leave for the rows' owners as bf16,
    per-tensor scales applied). ``row_ss_out`` [M, ceil(N / 256)] receives the sums of squares of the new rows."""
    M, N = a.rows, w.rows
    nv.ensure_splitk_workspace(a.device)
    g = _base_args(a, w, M, N, EPI_RESIDUAL, bn, 0, 0)
    g.out, g.ldo = x.data_ptr(), x.stride(0)
    g.residual, g.ldr, g.row_ss_out = x.data_ptr(), x.stride(0), row_ss_out.data_ptr()
    g.ar_world, g.ar_rank, g.ar_mc_base, g.ar_peer_base = world, rank, mc_base, peer_base
    g.ar_region_bytes, g.ar_recv_off, g.ar_recv_bytes = region_bytes, recv_off, recv_bytes
    g.ar_res_off, g.ar_res_bytes, g.ar_state = res_off, res_bytes, state
    nv.check(nv.lib().gllm_gemm_blockscaled(ctypes.byref(g)), "gemm_blockscaled_residual_allreduce")
    return row_ss_out


def gemm_glu(a: BlockScaled, w_packed: BlockScaled, *, act=0, out=None, row_ss=None, norm_dim=0, eps=0.0, bn: int = 128,
             mblk_group=None, num_groups: int = 0, splits: int = 0):
    """out[M, N/2] = act(rowscale * gate) * (rowscale * up); ``w_packed`` rows follow ``linear.interleave_gate_up``."""
    from .linear import _act_ref, deinterleave_gate_up, row_scale_ref
    M = a.rows
    N = w_packed.rows if mblk_group is None else w_packed.rows // num_groups
    if not a.codes.is_cuda:
        A, W = a.dequantize()[:M], w_packed.dequantize()
        rs = row_scale_ref(row_ss, norm_dim, eps)
        res = torch.zeros((M, N // 2), dtype=torch.bfloat16)
        groups = [(0, M, 0)] if mblk_group is None else [
            (i * 128, min(M, (i + 1) * 128), int(mblk_group[i])) for i in range((M + 127) // 128)]
        for r0, r1, gi in groups:
            if gi < 0:
                continue
            gw, uw = deinterleave_gate_up(W[gi * N:(gi + 1) * N])
            gv, uv = A[r0:r1] @ gw.t(), A[r0:r1] @ uw.t()
            if rs is not None:
                gv, uv = gv * rs[r0:r1, None], uv * rs[r0:r1, None]
            res[r0:r1] = (_act_ref(gv, act) * uv).to(torch.bfloat16)
        if out is not None:
            out.copy_(res)
            return out
        return res
    if out is None:
        out = torch.empty((M, N // 2), dtype=torch.bfloat16, device=a.device)
    nv.ensure_splitk_workspace(a.device)
    g = _base_args(a, w_packed, M, N, EPI_GLU, bn, 1 if mblk_group is not None else splits, 0)
    g.out, g.ldo, g.glu_act = out.data_ptr(), out.stride(0), act
    if row_ss is not None:
        g.row_ss_in, g.ss_in_parts = row_ss.data_ptr(), (row_ss.shape[1] if row_ss.dim() > 1 else 1)
        g.norm_inv_dim, g.norm_eps = 1.0 / norm_dim, eps
    if mblk_group is not None:
        g.mblk_group, g.num_groups = mblk_group.data_ptr(), num_groups
    nv.check(nv.lib().gllm_gemm_blockscaled(ctypes.byref(g)), "gemm_blockscaled_glu")
    return out


def gemm_qkv(a: BlockScaled, w_qkv: BlockScaled, *, n_q, n_kv, q_out, kv_cache, slot_mapping, positions, cos_t, sin_t,
             q_norm_w=None, k_norm_w=None, qk_eps=1e-6, row_ss=None, norm_dim=0, eps=0.0, bias=None, kv_scale=1.0,
             splits: int = 0):
    """Fused QKV projection (head_dim 128) on block-scaled operands: per-head norm, RoPE, q buffer and paged KV write."""
    from .linear import kv_write_ref, qkv_post_ref
    M = a.rows
    if not a.codes.is_cuda:
        acc = _ref_acc(a, w_qkv, M, row_ss, norm_dim, eps)
        if bias is not None:
            acc = acc + bias.float()
        q, k, v = qkv_post_ref(acc, n_q, n_kv, 128, positions, cos_t, sin_t, q_norm_w, k_norm_w, qk_eps)
        q_out[:M].copy_(q.reshape(M, n_q * 128).to(q_out.dtype))
        if slot_mapping is not None:
            kv_write_ref(kv_cache, k, v, slot_mapping, kv_scale)
        return q_out
    nv.ensure_splitk_workspace(a.device)
    g = _base_args(a, w_qkv, M, (n_q + 2 * n_kv) * 128, EPI_QKV, 128, splits, 0)
    g.bias = nv.ptr(bias)
    if row_ss is not None:
        g.row_ss_in, g.ss_in_parts = row_ss.data_ptr(), (row_ss.shape[1] if row_ss.dim() > 1 else 1)
        g.norm_inv_dim, g.norm_eps = 1.0 / norm_dim, eps
    g.n_q_heads, g.n_kv_heads, g.q_out, g.kv_cache = n_q, n_kv, q_out.data_ptr(), kv_cache.data_ptr()
    g.num_pages, g.slot_mapping, g.positions = kv_cache.shape[0], nv.ptr(slot_mapping), positions.data_ptr()
    g.cos_table, g.sin_table, g.max_pos = cos_t.data_ptr(), sin_t.data_ptr(), cos_t.shape[0]
    g.q_norm_w, g.k_norm_w, g.qk_eps = nv.ptr(q_norm_w), nv.ptr(k_norm_w), qk_eps
    g.kv_inv_scale = (1.0 / kv_scale) if kv_cache.dtype == torch.float8_e4m3fn else 0.0
    nv.check(nv.lib().gllm_gemm_blockscaled(ctypes.byref(g)), "gemm_blockscaled_qkv")
    return q_out
