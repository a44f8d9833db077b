"""Linear-layer ops: the tcgen05 GEMM family and its fused epilogues.

Every function has two paths: CUDA tensors go to the hand-written sm_100a kernel
(``csrc/kernels/gemm_sm100.cu``); CPU tensors go to an fp32 PyTorch restatement with the same
rounding points, which doubles as the numerical oracle in the tests.

Weight layout is the checkpoint's ``[out, in]`` row-major ("trans_b = true",
reference: src/arch/auto_graph_fragments/build_graph.inc.rs:1618).
"""
from __future__ import annotations

import torch

from . import _native as nv

PAGE = 16


def _bn_for(n: int, m: int) -> int:
    """Tile width: 256-wide tiles when they fill the machine, else 128."""
    if n % 256 == 0 and (n // 256) * ((m + 127) // 128) >= 120:
        return 256
    return 128


def pad_rows(w: torch.Tensor, multiple: int = 128) -> torch.Tensor:
    """Zero-pad the out-features of a weight to a multiple (done once at load time)."""
    n = w.shape[0]
    if n % multiple == 0:
        return w
    pad = multiple - n % multiple
    return torch.cat([w, w.new_zeros((pad,) + tuple(w.shape[1:]))], 0).contiguous()


GLU_GROUP = 64   # packed gate/up rows come in groups of 64: 32 gate rows, then the matching 32 up rows


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor, bn: int = 256) -> torch.Tensor:
    """Pack gate/up weights so that every 64 rows hold 32 gate rows followed by the matching 32 up rows.

    The GLU epilogue then finds both halves of an output feature inside one accumulator tile whatever the tile
    width (128, 192 or 256 columns are all multiples of 64), so the width can be chosen per call: wide tiles for
    prefill, a width that fills one wave of SMs for decode. ``bn`` is accepted for callers that record the decode
    tile width next to the weight; the packing does not depend on it. Requires intermediate size % 32 == 0.
    """
    inter, k = gate.shape
    half = GLU_GROUP // 2
    if inter % half != 0:
        raise ValueError(f"intermediate size {inter} must be a multiple of {half}")
    g = gate.reshape(inter // half, half, k)
    u = up.reshape(inter // half, half, k)
    return torch.stack([g, u], 1).reshape(2 * inter, k).contiguous()


def deinterleave_gate_up(w: torch.Tensor, bn: int = 256):
    half = GLU_GROUP // 2
    n, k = w.shape
    t = w.reshape(n // GLU_GROUP, 2, half, k)
    return t[:, 0].reshape(n // 2, k), t[:, 1].reshape(n // 2, k)


def _on_device(a, **tensors):
    """A host tensor handed to a device kernel is an illegal address on the GPU: refuse it on the host."""
    for name, t in tensors.items():
        if t is not None and t.device != a.device:
            raise ValueError(f"{name} is on {t.device} but the activations are on {a.device}")


def row_scale_ref(row_ss, norm_dim, eps):
    if row_ss is None:
        return None
    ss = row_ss.float().reshape(row_ss.shape[0], -1).sum(-1)
    return torch.rsqrt(ss / norm_dim + eps)


# --------------------------------------------------------------------------------------------
# plain GEMM (+ RMSNorm-as-row-scale prologue, + bias)
# --------------------------------------------------------------------------------------------
def gemm(a, w, *, out=None, out_dtype=torch.bfloat16, bias=None, row_ss=None, norm_dim=0, eps=0.0,
         bn=None, max_ctas=0, splits=0, softcap: float = 0.0):
    """out[M,N] = rowscale(a) @ w.T (+ bias). ``row_ss`` [M, parts] are partial sums of squares of ``a``'s
    rows; when given, each output row is scaled by rsqrt(sum/norm_dim + eps) (the norm weight must
    already be folded into ``w``). ``softcap`` > 0 applies cap * tanh(x / cap) to the result (final-logit soft
    capping) in the GEMM epilogue."""
    from .quant_gemm import QuantWeight, qgemm
    if isinstance(w, QuantWeight):      # quantised weight: dequantisation fused into the GEMM main loop
        y = qgemm(a, w, row_ss=row_ss, norm_dim=norm_dim, eps=eps)
        if bias is not None or out_dtype != y.dtype or softcap:
            y = y.float() + bias.float() if bias is not None else y.float()
            if softcap:
                y = torch.tanh(y / softcap) * softcap
            y = y.to(out_dtype)
        if out is not None:
            out.copy_(y)
            return out
        return y
    M, K = a.shape
    N = w.shape[0]
    if not a.is_cuda:
        acc = a.float() @ w.float().t()
        rs = row_scale_ref(row_ss, norm_dim, eps)
        if rs is not None:
            acc = acc * rs[:, None]
        if bias is not None:
            acc = acc + bias.float()
        if softcap:
            acc = torch.tanh(acc / softcap) * softcap
        res = acc.to(out.dtype if out is not None else out_dtype)
        if out is not None:
            out.copy_(res)
            return out
        return res
    assert a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
    assert a.stride(-1) == 1 and w.stride(-1) == 1
    _on_device(a, weight=w, bias=bias, row_ss=row_ss, out=out)
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=a.device)
    bn = bn or _bn_for(N, M)
    nv.ensure_splitk_workspace(a.device)
    parts = 0 if row_ss is None else (row_ss.shape[1] if row_ss.dim() > 1 else 1)
    if softcap:
        rc = nv.lib().gllm_gemm_bf16_softcap(a.data_ptr(), a.stride(0), w.data_ptr(), w.stride(0), out.data_ptr(),
                                             out.stride(0), M, N, K, 1 if out.dtype == torch.float32 else 0, nv.ptr(bias),
                                             nv.ptr(row_ss), parts, 1.0 / norm_dim if norm_dim else 0.0, eps, bn,
                                             nv.stream_ptr(), float(softcap))
        nv.check(rc, "gemm_bf16_softcap")
        return out
    rc = nv.lib().gllm_gemm_bf16(a.data_ptr(), a.stride(0), w.data_ptr(), w.stride(0), out.data_ptr(), out.stride(0),
                                 M, N, K, 1 if out.dtype == torch.float32 else 0, nv.ptr(bias), nv.ptr(row_ss),
                                 parts, 1.0 / norm_dim if norm_dim else 0.0, eps, bn, nv.stream_ptr(), max_ctas,
                                 splits)
    nv.check(rc, "gemm_bf16")
    return out


def gemm_residual(a, w, residual, *, out=None, row_ss_out=None, bias=None, bn=None, max_ctas=0, splits=0):
    """out = a @ w.T (+bias) + residual (bf16). Returns (out, row_ss) where row_ss[M, ceil(N/bn)] holds the
    per-tile sums of squares of ``out``: the next layer's RMSNorm statistics."""
    from .quant_gemm import QuantWeight, qgemm
    if isinstance(w, QuantWeight):
        from .elementwise import rmsnorm
        M = a.shape[0]
        y = qgemm(a, w)
        if bias is not None:
            y = (y.float() + bias.float()).to(y.dtype)
        out = residual if out is None else out
        ss = row_ss_out if row_ss_out is not None else torch.empty((M, 1), dtype=torch.float32, device=a.device)
        rmsnorm(y, None, 0.0, residual=residual, h_out=out, ss_out=ss, want_y=False)
        if ss.dim() > 1 and ss.shape[1] > 1:      # statistics land in column 0; the other tile columns are zero
            flat = ss.reshape(-1)[:M].clone()
            ss[:M].zero_()
            ss[:M, 0] = flat
        return out, ss
    M, K = a.shape
    N = w.shape[0]
    bn = bn or _bn_for(N, M)
    parts = (N + bn - 1) // bn
    if not a.is_cuda:
        acc = a.float() @ w.float().t()
        if bias is not None:
            acc = acc + bias.float()
        res = (acc + residual.float()).to(a.dtype)
        ss = res.float().pow(2)
        pad = parts * bn - N
        if pad:
            ss = torch.nn.functional.pad(ss, (0, pad))
        ss = ss.reshape(M, parts, bn).sum(-1)
        if out is not None:
            out.copy_(res)
            res = out
        if row_ss_out is not None:
            row_ss_out[:M, :parts].copy_(ss)
            ss = row_ss_out
        return res, ss
    _on_device(a, weight=w, residual=residual, bias=bias, out=out, row_ss_out=row_ss_out)
    if out is None:
        out = torch.empty((M, N), dtype=torch.bfloat16, device=a.device)
    if row_ss_out is None:
        row_ss_out = torch.empty((M, parts), dtype=torch.float32, device=a.device)
    assert row_ss_out.shape[-1] == parts and row_ss_out.is_contiguous()
    nv.ensure_splitk_workspace(a.device)
    rc = nv.lib().gllm_gemm_bf16_residual(a.data_ptr(), a.stride(0), w.data_ptr(), w.stride(0), out.data_ptr(),
                                          out.stride(0), residual.data_ptr(), residual.stride(0),
                                          row_ss_out.data_ptr(), M, N, K, nv.ptr(bias), bn, nv.stream_ptr(), max_ctas,
                                          splits)
    nv.check(rc, "gemm_bf16_residual")
    return out, row_ss_out


def set_pair_max_m(max_m: int, epi_mask: int = 0xF):
    """GEMMs with 128 < M <= ``max_m`` whose epilogue is in ``epi_mask`` (bit 0 store, 1 residual, 2 GLU, 3 QKV) run on
    CTA pairs (`tcgen05.mma.cta_group::2`, clusters of two); ``max_m`` 0 turns the path off. Returns the previous
    ``(max_m, epi_mask)`` so a caller can restore it."""
    old = int(nv.lib().gllm_gemm_set_pair(int(max_m), int(epi_mask)))
    return old & 0xFFFF, old >> 16


def set_pair_big_m(big_m: int) -> int:
    """256-wide GEMMs with M >= ``big_m`` run on CTA pairs (0 = never). Returns the previous threshold."""
    return int(nv.lib().gllm_gemm_set_pair_big_m(int(big_m)))


ACT_IDS = {"silu": 0, "swiglu": 0, "gelu_tanh": 1, "gelu_new": 1, "gelu_pytorch_tanh": 1, "geglu": 1, "gelu": 1}


def _act_ref(g, act):
    if act == 0:
        return torch.nn.functional.silu(g)
    return torch.nn.functional.gelu(g, approximate="tanh")


def gemm_glu(a, w_packed, *, act=0, out=None, row_ss=None, norm_dim=0, eps=0.0, bn=256, mblk_group=None,
             num_groups=0, max_ctas=0, splits=0):
    """out[M, N/2] = act(rowscale*gate) * (rowscale*up) with gate/up packed by ``interleave_gate_up``.
    With ``mblk_group`` (int32 per 128-row block) the weight is a stack of per-expert matrices."""
    M, K = a.shape
    if mblk_group is None:
        N = w_packed.shape[0]
    else:
        N = w_packed.shape[0] // num_groups
    if not a.is_cuda:
        rs = row_scale_ref(row_ss, norm_dim, eps)
        res = torch.zeros((M, N // 2), dtype=a.dtype)
        groups = [(0, M, 0)] if mblk_group is None else [
            (i * 128, min(M, (i + 1) * 128), int(mblk_group[i])) for i in range((M + 127) // 128)]
        for (r0, r1, g) in groups:
            if g < 0:  # inactive row block of a grouped launch
                continue
            wg = w_packed[g * N:(g + 1) * N]
            gw, uw = deinterleave_gate_up(wg, bn)
            x = a[r0:r1].float()
            gv, uv = x @ gw.float().t(), x @ uw.float().t()
            if rs is not None:
                gv, uv = gv * rs[r0:r1, None], uv * rs[r0:r1, None]
            res[r0:r1] = (_act_ref(gv, act) * uv).to(a.dtype)
        if out is not None:
            out.copy_(res)
            return out
        return res
    _on_device(a, weight=w_packed, row_ss=row_ss, out=out, mblk_group=mblk_group)
    if out is None:
        out = torch.empty((M, N // 2), dtype=torch.bfloat16, device=a.device)
    parts = 0 if row_ss is None else (row_ss.shape[1] if row_ss.dim() > 1 else 1)
    nv.ensure_splitk_workspace(a.device)
    rc = nv.lib().gllm_gemm_bf16_glu(a.data_ptr(), a.stride(0), w_packed.data_ptr(), w_packed.stride(0),
                                     out.data_ptr(), out.stride(0), M, N, K, act, nv.ptr(row_ss), parts,
                                     1.0 / norm_dim if norm_dim else 0.0, eps, bn, nv.ptr(mblk_group), num_groups,
                                     nv.stream_ptr(), max_ctas, 1 if mblk_group is not None else splits)
    nv.check(rc, "gemm_bf16_glu")
    return out


def set_block_rows(rows):
    """Row counts of the 128-row blocks of the NEXT grouped GEMM launched by this thread (``MoeWorkspace.blk_rows``):
    the kernel then loads and stores only the rows that exist. No-op for CPU tensors."""
    if rows is not None and rows.is_cuda:
        nv.check(nv.lib().gllm_gemm_set_block_rows(rows.data_ptr()), "gemm_set_block_rows")


def gemm_grouped(a, w_stack, mblk_group, num_groups, *, out=None, bn=128, max_ctas=0):
    """Grouped GEMM: rows [128i, 128i+128) of ``a`` multiply expert ``mblk_group[i]``'s [N,K] weight."""
    M, K = a.shape
    N = w_stack.shape[0] // num_groups
    if not a.is_cuda:
        res = torch.zeros((M, N), dtype=a.dtype)
        for i in range((M + 127) // 128):
            g = int(mblk_group[i])
            if g < 0:
                continue
            res[i * 128:(i + 1) * 128] = (a[i * 128:(i + 1) * 128].float() @ w_stack[g * N:(g + 1) * N].float().t()).to(a.dtype)
        if out is not None:
            out.copy_(res)
            return out
        return res
    _on_device(a, weight=w_stack, mblk_group=mblk_group, out=out)
    if out is None:
        out = torch.empty((M, N), dtype=torch.bfloat16, device=a.device)
    rc = nv.lib().gllm_gemm_bf16_grouped(a.data_ptr(), a.stride(0), w_stack.data_ptr(), w_stack.stride(0),
                                         out.data_ptr(), out.stride(0), M, N, K, mblk_group.data_ptr(), num_groups,
                                         bn, nv.stream_ptr(), max_ctas)
    nv.check(rc, "gemm_bf16_grouped")
    return out


# --------------------------------------------------------------------------------------------
# fused QKV: GEMM -> per-head RMSNorm -> RoPE -> q buffer / paged KV write (head_dim 128)
# --------------------------------------------------------------------------------------------
def rope_ref(x, cos, sin):
    """Half-split (NeoX) rotation of the first 2*cos.shape[-1] features (scalar_ops.rs:42-63)."""
    half = cos.shape[-1]
    x1, x2, rest = x[..., :half], x[..., half:2 * half], x[..., 2 * half:]
    return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin, rest], -1)


def qkv_post_ref(qkv, n_q, n_kv, D, positions, cos_t, sin_t, q_norm_w, k_norm_w, qk_eps):
    """fp32 reference of the QKV epilogue; returns q [M,n_q,D], k [M,n_kv,D], v [M,n_kv,D] in fp32."""
    M = qkv.shape[0]
    x = qkv.float().reshape(M, n_q + 2 * n_kv, D)
    q, k, v = x[:, :n_q], x[:, n_q:n_q + n_kv], x[:, n_q + n_kv:]
    if q_norm_w is not None:
        q = q * torch.rsqrt(q.pow(2).mean(-1, keepdim=True) + qk_eps) * q_norm_w.float()
    if k_norm_w is not None:
        k = k * torch.rsqrt(k.pow(2).mean(-1, keepdim=True) + qk_eps) * k_norm_w.float()
    if cos_t is not None:
        cos = cos_t[positions.long()].float()[:, None, :]
        sin = sin_t[positions.long()].float()[:, None, :]
        q, k = rope_ref(q, cos, sin), rope_ref(k, cos, sin)
    return q, k, v


def kv_write_ref(kv_cache, k, v, slot_mapping, kv_scale: float = 1.0):
    """kv_cache: [pages, 2, n_kv, 16, D]; an fp8 cache stores value / kv_scale (saturating)."""
    slots = slot_mapping.long()
    ok = slots >= 0
    pages, offs = slots[ok] // PAGE, slots[ok] % PAGE
    if kv_cache.dtype == torch.float8_e4m3fn:
        enc = lambda t: (t[ok].float() / kv_scale).clamp(-448.0, 448.0).to(torch.float8_e4m3fn).view(torch.uint8)
        raw = kv_cache.view(torch.uint8)
        raw[pages, 0, :, offs] = enc(k)
        raw[pages, 1, :, offs] = enc(v)
        return
    kv_cache[pages, 0, :, offs] = k[ok].to(kv_cache.dtype)
    kv_cache[pages, 1, :, offs] = v[ok].to(kv_cache.dtype)


def gemm_qkv(a, w_qkv, *, n_q, n_kv, q_out, kv_cache, slot_mapping, positions, cos_t, sin_t, q_norm_w=None,
             k_norm_w=None, qk_eps=1e-6, row_ss=None, norm_dim=0, eps=0.0, bias=None, max_ctas=0, splits=0,
             kv_scale: float = 1.0):
    """Fused QKV projection for head_dim 128. ``w_qkv`` rows: q heads, k heads, v heads. An fp8 (e4m3) ``kv_cache``
    receives value / kv_scale."""
    M, K = a.shape
    D = 128
    if not a.is_cuda:
        acc = a.float() @ w_qkv.float().t()
        rs = row_scale_ref(row_ss, norm_dim, eps)
        if rs is not None:
            acc = acc * rs[:, None]
        if bias is not None:
            acc = acc + bias.float()
        q, k, v = qkv_post_ref(acc, n_q, n_kv, D, positions, cos_t, sin_t, q_norm_w, k_norm_w, qk_eps)
        q_out[:M].copy_(q.reshape(M, n_q * D).to(q_out.dtype))
        if slot_mapping is not None:
            kv_write_ref(kv_cache, k, v, slot_mapping, kv_scale)
        return q_out
    _on_device(a, weight=w_qkv, q_out=q_out, kv_cache=kv_cache, slot_mapping=slot_mapping, positions=positions,
               cos=cos_t, sin=sin_t, q_norm=q_norm_w, k_norm=k_norm_w, row_ss=row_ss, bias=bias)
    parts = 0 if row_ss is None else (row_ss.shape[1] if row_ss.dim() > 1 else 1)
    nv.ensure_splitk_workspace(a.device)
    if kv_cache.dtype == torch.float8_e4m3fn:
        rc = nv.lib().gllm_gemm_bf16_qkv_fp8kv(
            a.data_ptr(), a.stride(0), w_qkv.data_ptr(), w_qkv.stride(0), M, K, n_q, n_kv, q_out.data_ptr(),
            kv_cache.data_ptr(), kv_cache.shape[0], nv.ptr(slot_mapping), positions.data_ptr(), cos_t.data_ptr(),
            sin_t.data_ptr(), cos_t.shape[0], nv.ptr(q_norm_w), nv.ptr(k_norm_w), qk_eps, nv.ptr(row_ss), parts,
            1.0 / norm_dim if norm_dim else 0.0, eps, nv.ptr(bias), float(kv_scale), nv.stream_ptr(), max_ctas, splits)
        nv.check(rc, "gemm_bf16_qkv_fp8kv")
        return q_out
    rc = nv.lib().gllm_gemm_bf16_qkv(a.data_ptr(), a.stride(0), w_qkv.data_ptr(), w_qkv.stride(0), M, K, n_q, n_kv,
                                     q_out.data_ptr(), kv_cache.data_ptr(), kv_cache.shape[0], nv.ptr(slot_mapping),
                                     positions.data_ptr(), cos_t.data_ptr(), sin_t.data_ptr(), cos_t.shape[0],
                                     nv.ptr(q_norm_w), nv.ptr(k_norm_w), qk_eps, nv.ptr(row_ss), parts,
                                     1.0 / norm_dim if norm_dim else 0.0, eps, nv.ptr(bias), nv.stream_ptr(),
                                     max_ctas, splits)
    nv.check(rc, "gemm_bf16_qkv")
    return q_out


# --------------------------------------------------------------------------------------------
# FP8 e4m3 GEMM with per-row / per-column scales
# --------------------------------------------------------------------------------------------
def gemm_fp8(a8, w8, a_scale, b_scale, *, out=None, out_dtype=torch.bfloat16, bn=None, max_ctas=0, splits=0):
    M, K = a8.shape
    N = w8.shape[0]
    if not a8.is_cuda:
        acc = a8.float() @ w8.float().t()
        if a_scale is not None:
            acc = acc * a_scale.float()[:, None]
        if b_scale is not None:
            acc = acc * b_scale.float()[None, :]
        res = acc.to(out_dtype)
        if out is not None:
            out.copy_(res)
            return out
        return res
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=a8.device)
    bn = bn or _bn_for(N, M)
    nv.ensure_splitk_workspace(a8.device)
    rc = nv.lib().gllm_gemm_fp8(a8.data_ptr(), a8.stride(0), w8.data_ptr(), w8.stride(0), out.data_ptr(),
                                out.stride(0), M, N, K, 1 if out.dtype == torch.float32 else 0, nv.ptr(a_scale),
                                nv.ptr(b_scale), bn, nv.stream_ptr(), max_ctas, splits)
    nv.check(rc, "gemm_fp8")
    return out
