"""Paged attention ops over the 16-token-page KV cache ``[pages, 2, n_kv, 16, D]``.

CUDA path: ``csrc/kernels/attention.cu`` (head_dim 128, TMA page gathers + tensor-core math) or the
generic kernel in ``misc.cu`` for other head dims. CPU path / oracle: plain fp32 softmax attention with the
reference's semantics (src/compat/scalar_ops.rs:196-278,316-378): scale 1/sqrt(d), GQA head mapping
``kv_h = h // (Hq/Hkv)``, causal mask, max-subtracted softmax, optional sliding window and sinks.
"""
from __future__ import annotations

import math

import torch

from . import _native as nv

PAGE = 16


def gather_kv_ref(kv_cache, block_table, ctx_len):
    """Return K, V as [ctx_len, n_kv, D] fp32 for one sequence."""
    n_pages = (ctx_len + PAGE - 1) // PAGE
    pages = block_table[:n_pages].long()
    k = kv_cache[pages, 0].permute(0, 2, 1, 3).reshape(n_pages * PAGE, kv_cache.shape[2], kv_cache.shape[4])
    v = kv_cache[pages, 1].permute(0, 2, 1, 3).reshape(n_pages * PAGE, kv_cache.shape[2], kv_cache.shape[4])
    return k[:ctx_len].float(), v[:ctx_len].float()


def _dequant_cache(kv_cache, kv_scale):
    """fp8 cache -> fp32 values (oracle path)."""
    return kv_cache.float() * kv_scale if kv_cache.dtype == torch.float8_e4m3fn else kv_cache


def attention_ref(q, kv_cache, block_tables, q_start, q_len, ctx_lens, n_q, n_kv, scale, causal=True, window=0,
                  sinks=None):
    """q: [T, n_q*D]. Returns [T, n_q*D] in q.dtype. Works on any device (used as the oracle)."""
    D = kv_cache.shape[-1]
    out = torch.zeros_like(q)
    group = n_q // n_kv
    for s in range(len(q_len)):
        ql, ctx, st = int(q_len[s]), int(ctx_lens[s]), int(q_start[s])
        if ql <= 0 or ctx <= 0:
            continue
        k, v = gather_kv_ref(kv_cache, block_tables[s], ctx)
        qs = q[st:st + ql].float().reshape(ql, n_q, D)
        kk = k.repeat_interleave(group, 1)  # [ctx, n_q, D]
        vv = v.repeat_interleave(group, 1)
        scores = torch.einsum("qhd,khd->hqk", qs, kk) * scale
        pos_q = torch.arange(ctx - ql, ctx, device=q.device)[:, None]
        pos_k = torch.arange(ctx, device=q.device)[None, :]
        mask = torch.ones((ql, ctx), dtype=torch.bool, device=q.device)
        if causal:
            mask &= pos_k <= pos_q
            if window > 0:
                mask &= pos_k > pos_q - window
        elif window > 0:
            mask &= pos_k >= ctx - window
        scores = scores.masked_fill(~mask[None], float("-inf"))
        if sinks is not None:
            sk = sinks.float().reshape(n_q, 1, 1).expand(n_q, ql, 1)
            probs = torch.softmax(torch.cat([scores, sk], -1), -1)[..., :-1]
        else:
            probs = torch.softmax(scores, -1)
        o = torch.einsum("hqk,khd->qhd", probs, vv)
        out[st:st + ql] = o.reshape(ql, n_q * D).to(q.dtype)
    return out


class DecodeWorkspace:
    """Scratch for split-KV decode (partial outputs, log-sum-exps and the ticket counters)."""

    def __init__(self, max_batch, n_q, n_kv, max_splits, device):
        self.max_batch, self.max_splits = max_batch, max_splits
        n = nv.lib().gllm_decode_scratch_floats(max_batch, n_q, max_splits) if device.type == "cuda" else 1
        self.scratch = torch.empty(int(n), dtype=torch.float32, device=device)
        self.counters = torch.zeros(max_batch * n_kv, dtype=torch.int32, device=device)


def paged_decode(q, kv_cache, block_tables, ctx_lens, *, n_q, n_kv, scale=None, out=None, workspace=None,
                 pages_per_split=32, window=0, sinks=None, kv_scale: float = 1.0):
    """One query token per sequence. q: [B, n_q*D]; ctx_lens includes the token just written."""
    B = q.shape[0]
    D = kv_cache.shape[-1]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    if out is None:
        out = torch.empty_like(q)
    if not q.is_cuda:
        ar = torch.arange(B, dtype=torch.int32)
        ones = (ctx_lens > 0).to(torch.int32)
        out.copy_(attention_ref(q, _dequant_cache(kv_cache, kv_scale), block_tables, ar, ones, ctx_lens, n_q, n_kv, scale,
                                True, window, sinks))
        return out
    if D == 128 and n_q // n_kv <= 16:
        max_blocks = block_tables.shape[1]
        if workspace is None:
            max_splits = max(1, (max_blocks + pages_per_split - 1) // pages_per_split)
            workspace = DecodeWorkspace(B, n_q, n_kv, max_splits, q.device)
        if kv_cache.dtype == torch.float8_e4m3fn:     # same TMA / tensor-core kernel, fp8 pages converted in registers
            rc = nv.lib().gllm_paged_decode_fp8(q.data_ptr(), out.data_ptr(), kv_cache.data_ptr(), kv_cache.shape[0],
                                                block_tables.data_ptr(), max_blocks, ctx_lens.data_ptr(), B, n_q, n_kv,
                                                scale, pages_per_split, workspace.max_splits,
                                                workspace.scratch.data_ptr(), workspace.counters.data_ptr(), window,
                                                nv.ptr(sinks), float(kv_scale), nv.stream_ptr())
            nv.check(rc, "paged_decode_fp8")
            return out
        rc = nv.lib().gllm_paged_decode(q.data_ptr(), out.data_ptr(), kv_cache.data_ptr(), kv_cache.shape[0],
                                        block_tables.data_ptr(), max_blocks, ctx_lens.data_ptr(), B, n_q, n_kv,
                                        scale, pages_per_split, workspace.max_splits, workspace.scratch.data_ptr(),
                                        workspace.counters.data_ptr(), window, nv.ptr(sinks), nv.stream_ptr())
        nv.check(rc, "paged_decode")
        return out
    ar = torch.arange(B, dtype=torch.int32, device=q.device)
    ones = (ctx_lens > 0).to(torch.int32)
    return paged_prefill(q, kv_cache, block_tables, ar, ones, ctx_lens, max_q_len=1, n_q=n_q, n_kv=n_kv, scale=scale,
                         out=out, window=window, kv_scale=kv_scale)


def paged_prefill(q, kv_cache, block_tables, q_start, q_len, ctx_lens, *, max_q_len, n_q, n_kv, scale=None,
                  out=None, causal=True, window=0, sinks=None, kv_scale: float = 1.0):
    """Variable-length (chunked) prefill. q: [T, n_q*D] flat tokens; sequence i owns rows
    [q_start[i], q_start[i]+q_len[i]) which are the last q_len[i] of its ctx_lens[i] cached tokens."""
    D = kv_cache.shape[-1]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    if out is None:
        out = torch.empty_like(q)
    if not q.is_cuda:
        out.copy_(attention_ref(q, _dequant_cache(kv_cache, kv_scale), block_tables, q_start, q_len, ctx_lens, n_q, n_kv, scale,
                                causal, window, sinks))
        return out
    S = q_len.shape[0]
    if kv_cache.dtype == torch.float8_e4m3fn and D == 128:
        rc = nv.lib().gllm_paged_prefill_fp8(q.data_ptr(), out.data_ptr(), kv_cache.data_ptr(), kv_cache.shape[0],
                                             block_tables.data_ptr(), block_tables.shape[1], q_start.data_ptr(),
                                             q_len.data_ptr(), ctx_lens.data_ptr(), S, max_q_len, n_q, n_kv, scale,
                                             1 if causal else 0, window, nv.ptr(sinks), float(kv_scale), nv.stream_ptr())
        nv.check(rc, "paged_prefill_fp8")
        return out
    if kv_cache.dtype == torch.float8_e4m3fn:
        if sinks is not None:
            raise NotImplementedError("attention sinks with an fp8 KV cache")
        rc = nv.lib().gllm_paged_attention_fp8kv(q.data_ptr(), out.data_ptr(), kv_cache.data_ptr(), kv_cache.shape[0],
                                                 block_tables.data_ptr(), block_tables.shape[1], q_start.data_ptr(),
                                                 q_len.data_ptr(), ctx_lens.data_ptr(), S, max_q_len, n_q, n_kv, D, scale,
                                                 1 if causal else 0, window, float(kv_scale), nv.stream_ptr())
        nv.check(rc, "paged_attention_fp8kv")
        return out
    if D == 128 and nv.get_option("prefill_tc") != 0 and q.is_contiguous() and out.is_contiguous():
        # tcgen05 flash attention (S and O accumulators in tensor memory)
        rc = nv.lib().gllm_paged_prefill_tc(q.data_ptr(), out.data_ptr(), kv_cache.data_ptr(), kv_cache.shape[0],
                                            block_tables.data_ptr(), block_tables.shape[1], q_start.data_ptr(),
                                            q_len.data_ptr(), ctx_lens.data_ptr(), S, max_q_len, q.shape[0], n_q, n_kv,
                                            scale, 1 if causal else 0, window, nv.ptr(sinks), nv.stream_ptr())
        nv.check(rc, "paged_prefill_tc")
    elif D == 128:
        rc = nv.lib().gllm_paged_prefill(q.data_ptr(), out.data_ptr(), kv_cache.data_ptr(), kv_cache.shape[0],
                                         block_tables.data_ptr(), block_tables.shape[1], q_start.data_ptr(),
                                         q_len.data_ptr(), ctx_lens.data_ptr(), S, max_q_len, n_q, n_kv, scale,
                                         1 if causal else 0, window, nv.ptr(sinks), nv.stream_ptr())
        nv.check(rc, "paged_prefill")
    else:
        if sinks is not None:
            raise NotImplementedError("attention sinks need head_dim 128")
        rc = nv.lib().gllm_paged_attention_generic(q.data_ptr(), out.data_ptr(), kv_cache.data_ptr(),
                                                   kv_cache.shape[0], block_tables.data_ptr(), block_tables.shape[1],
                                                   q_start.data_ptr(), q_len.data_ptr(), ctx_lens.data_ptr(), S,
                                                   max_q_len, n_q, n_kv, D, scale, 1 if causal else 0, window,
                                                   nv.stream_ptr())
        nv.check(rc, "paged_attention_generic")
    return out
