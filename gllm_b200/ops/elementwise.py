"""Bandwidth-bound ops: embedding gather, norms, GLU, standalone RoPE + KV write, pooling, sampling.

CUDA path: ``csrc/kernels/misc.cu``. CPU path / oracle: fp32 PyTorch with the reference's semantics
(src/compat/scalar_ops.rs:11-63, src/compat/sampling.rs:28-135).
"""
from __future__ import annotations

import torch

from . import _native as nv
from .linear import kv_write_ref, qkv_post_ref


def embed_gather(ids, table, *, scale=1.0, out=None, ss_out=None):
    """out[m] = table[ids[m]] * scale; ss_out[m] = sum(out[m]^2) (RMSNorm statistics for the first layer)."""
    M = ids.shape[0]
    hidden = table.shape[1]
    if out is None:
        out = torch.empty((M, hidden), dtype=table.dtype, device=table.device)
    if not table.is_cuda:
        v = table[ids.long()]
        if scale != 1.0:
            v = (v.float() * scale).to(table.dtype)
        out.copy_(v)
        if ss_out is not None:
            ss_out.reshape(-1)[:M].copy_(out.float().pow(2).sum(-1))
        return out
    rc = nv.lib().gllm_embed_gather(ids.data_ptr(), table.data_ptr(), table.shape[0], hidden, float(scale),
                                    out.data_ptr(), nv.ptr(ss_out), M, nv.stream_ptr())
    nv.check(rc, "embed_gather")
    return out


def rmsnorm(x, w, eps, *, residual=None, one_plus_w=False, out=None, h_out=None, ss_out=None, want_y=True):
    """h = x (+residual); y = h * rsqrt(mean(h^2)+eps) * w. Returns y (or None if want_y is False).
    ``h_out`` receives h, ``ss_out`` the per-row sum of squares of h."""
    M, hidden = x.shape
    if not x.is_cuda:
        h = x.float()
        if residual is not None:
            h = (h + residual.float()).to(x.dtype).float()
        if h_out is not None:
            h_out.copy_(h.to(h_out.dtype))
        if ss_out is not None:
            ss_out.reshape(-1)[:M].copy_(h.pow(2).sum(-1))
        if not want_y:
            return None
        g = 1.0 if w is None else ((1.0 + w.float()) if one_plus_w else w.float())
        y = (h * torch.rsqrt(h.pow(2).mean(-1, keepdim=True) + eps) * g).to(x.dtype)
        if out is not None:
            out.copy_(y)
            return out
        return y
    if want_y and out is None:
        out = torch.empty_like(x)
    rc = nv.lib().gllm_rmsnorm(x.data_ptr(), nv.ptr(residual), nv.ptr(w), M, hidden, eps, 1 if one_plus_w else 0,
                               nv.ptr(h_out), out.data_ptr() if want_y else None, nv.ptr(ss_out), nv.stream_ptr())
    nv.check(rc, "rmsnorm")
    return out if want_y else None


def layernorm(x, w, b, eps, *, residual=None, out=None):
    M, hidden = x.shape
    if not x.is_cuda:
        h = x.float() if residual is None else x.float() + residual.float()
        y = torch.nn.functional.layer_norm(h, (hidden,), None if w is None else w.float(),
                                           None if b is None else b.float(), eps).to(x.dtype)
        if out is not None:
            out.copy_(y)
            return out
        return y
    if out is None:
        out = torch.empty_like(x)
    rc = nv.lib().gllm_layernorm(x.data_ptr(), nv.ptr(residual), nv.ptr(w), nv.ptr(b), M, hidden, eps, out.data_ptr(),
                                 nv.stream_ptr())
    nv.check(rc, "layernorm")
    return out


def glu(gu, act=0, *, out=None):
    """gu: [M, 2I] (gate | up) -> act(gate) * up. act: 0 silu, 1 gelu_tanh, 2 gelu_erf."""
    M, two_i = gu.shape
    inter = two_i // 2
    if not gu.is_cuda:
        g, u = gu[:, :inter].float(), gu[:, inter:].float()
        a = torch.nn.functional.silu(g) if act == 0 else torch.nn.functional.gelu(
            g, approximate="tanh" if act == 1 else "none")
        y = (a * u).to(gu.dtype)
        if out is not None:
            out.copy_(y)
            return out
        return y
    if out is None:
        out = torch.empty((M, inter), dtype=gu.dtype, device=gu.device)
    rc = nv.lib().gllm_glu(gu.data_ptr(), gu.stride(0), M, inter, act, out.data_ptr(), nv.stream_ptr())
    nv.check(rc, "glu")
    return out


def rope_kv_write(qkv, *, n_q, n_kv, head_dim, rot_dim, positions, slot_mapping, cos_t, sin_t, q_out, kv_cache,
                  q_norm_w=None, k_norm_w=None, qk_eps=1e-6, kv_scale: float = 1.0):
    """Unfused counterpart of the QKV epilogue for any head_dim: per-head norm -> RoPE -> q buffer / KV pages."""
    M = qkv.shape[0]
    if not qkv.is_cuda:
        q, k, v = qkv_post_ref(qkv, n_q, n_kv, head_dim, positions, cos_t if rot_dim > 0 else None, sin_t, q_norm_w,
                               k_norm_w, qk_eps)
        q_out[:M].copy_(q.reshape(M, n_q * head_dim).to(q_out.dtype))
        if slot_mapping is not None:
            kv_write_ref(kv_cache, k, v, slot_mapping, kv_scale)
        return q_out
    if kv_cache.dtype == torch.float8_e4m3fn:
        rc = nv.lib().gllm_rope_kv_write_fp8(qkv.data_ptr(), qkv.stride(0), M, n_q, n_kv, head_dim, rot_dim,
                                             positions.data_ptr(), nv.ptr(slot_mapping), nv.ptr(cos_t), nv.ptr(sin_t),
                                             cos_t.shape[0] if cos_t is not None else 1, nv.ptr(q_norm_w), nv.ptr(k_norm_w),
                                             qk_eps, q_out.data_ptr(), kv_cache.data_ptr(), kv_cache.shape[0], float(kv_scale),
                                             nv.stream_ptr())
        nv.check(rc, "rope_kv_write_fp8")
        return q_out
    rc = nv.lib().gllm_rope_kv_write(qkv.data_ptr(), qkv.stride(0), M, n_q, n_kv, head_dim, rot_dim,
                                     positions.data_ptr(), nv.ptr(slot_mapping), nv.ptr(cos_t), nv.ptr(sin_t),
                                     cos_t.shape[0] if cos_t is not None else 1, nv.ptr(q_norm_w), nv.ptr(k_norm_w),
                                     qk_eps, q_out.data_ptr(), kv_cache.data_ptr(), kv_cache.shape[0],
                                     nv.stream_ptr())
    nv.check(rc, "rope_kv_write")
    return q_out


def pool(h, seq_start, seq_len, mode="mean"):
    """Per-sequence pooling of flat hidden states [T, H] -> [S, H] fp32. mode: mean | cls | last."""
    m = {"mean": 0, "cls": 1, "last": 2}[mode]
    S = seq_len.shape[0]
    out = torch.empty((S, h.shape[1]), dtype=torch.float32, device=h.device)
    if not h.is_cuda:
        for s in range(S):
            st, n = int(seq_start[s]), int(seq_len[s])
            seg = h[st:st + n].float()
            out[s] = seg.mean(0) if m == 0 else (seg[0] if m == 1 else seg[-1])
        return out
    rc = nv.lib().gllm_pool(h.data_ptr(), seq_start.data_ptr(), seq_len.data_ptr(), S, h.shape[1], m, out.data_ptr(),
                            nv.stream_ptr())
    nv.check(rc, "pool")
    return out


# --------------------------------------------------------------------------------------------
# sampling
# --------------------------------------------------------------------------------------------
def argmax(logits, vocab=None, *, out=None, out_vals=None):
    """Row argmax over the first ``vocab`` columns; NaN never wins; lowest index wins ties."""
    B = logits.shape[0]
    vocab = vocab or logits.shape[1]
    if out is None:
        out = torch.empty(B, dtype=torch.int32, device=logits.device)
    if not logits.is_cuda:
        lg = logits[:, :vocab].float()
        lg = torch.where(torch.isnan(lg), torch.full_like(lg, float("-inf")), lg)
        vals, idx = lg.max(-1)
        out.copy_(idx.to(torch.int32))
        if out_vals is not None:
            out_vals.copy_(vals)
        return out
    rc = nv.lib().gllm_argmax(logits.data_ptr(), logits.stride(0), 1 if logits.dtype == torch.bfloat16 else 0, B,
                              vocab, out.data_ptr(), nv.ptr(out_vals), nv.stream_ptr())
    nv.check(rc, "argmax")
    return out


def sample_ref(logits_row, temperature, top_k, top_p, u):
    """The reference's order of operations on one row (src/compat/sampling.rs:28-135); ``u`` in [0,1)."""
    lg = logits_row.float()
    lg = torch.where(torch.isnan(lg), torch.full_like(lg, float("-inf")), lg)
    if temperature <= 0:
        return int(lg.argmax())
    vals, idx = torch.sort(lg, descending=True, stable=True)
    if 0 < top_k < vals.numel():
        vals, idx = vals[:top_k], idx[:top_k]
    probs = torch.softmax(vals / temperature, -1)
    if 0 < top_p < 1:
        cum = torch.cumsum(probs, -1)
        cut = int((cum >= top_p).nonzero()[0]) + 1 if bool((cum >= top_p).any()) else probs.numel()
        probs, idx = probs[:cut], idx[:cut]
        probs = probs / probs.sum()
    cum = torch.cumsum(probs, -1)
    j = int((cum > u).nonzero()[0]) if bool((cum > u).any()) else probs.numel() - 1
    return int(idx[j])


def filtered_probs_ref(logits_row, temperature, top_k, top_p):
    """Distribution the sampler draws from (dense vector over the vocabulary)."""
    lg = logits_row.float()
    vals, idx = torch.sort(lg, descending=True, stable=True)
    if 0 < top_k < vals.numel():
        vals, idx = vals[:top_k], idx[:top_k]
    probs = torch.softmax(vals / temperature, -1)
    if 0 < top_p < 1:
        cum = torch.cumsum(probs, -1)
        cut = int((cum >= top_p).nonzero()[0]) + 1 if bool((cum >= top_p).any()) else probs.numel()
        probs, idx = probs[:cut], idx[:cut]
        probs = probs / probs.sum()
    dense = torch.zeros_like(lg)
    dense[idx] = probs
    return dense


def sample(logits, params, *, vocab=None, seed=0, step_offsets=None, out=None, out_logprob=None, generator=None):
    """params: [B,4] fp32 rows {temperature, top_k, top_p, 0}. Returns int32 token ids [B]."""
    B = logits.shape[0]
    vocab = vocab or logits.shape[1]
    if out is None:
        out = torch.empty(B, dtype=torch.int32, device=logits.device)
    if not logits.is_cuda:
        for b in range(B):
            t, k, p = float(params[b, 0]), int(params[b, 1]), float(params[b, 2])
            gen = generator
            if gen is None and step_offsets is not None:
                # counter-based like the device sampler: the draw depends on (seed, row, the row's step counter) only,
                # so tensor-parallel ranks sampling the same row agree
                gen = torch.Generator().manual_seed((int(seed) * 1000003 + int(step_offsets[b]) * 7919 + b) & 0x7FFFFFFFFFFF)
            u = float(torch.rand((), generator=gen)) if t > 0 else 0.0
            out[b] = sample_ref(logits[b, :vocab], t, k, p, u)
        return out
    rc = nv.lib().gllm_sample(logits.data_ptr(), logits.stride(0), 1 if logits.dtype == torch.bfloat16 else 0, B, vocab,
                              params.data_ptr(), int(seed) & 0xFFFFFFFFFFFFFFFF, nv.ptr(step_offsets), out.data_ptr(),
                              nv.ptr(out_logprob), nv.stream_ptr())
    nv.check(rc, "sample")
    return out
