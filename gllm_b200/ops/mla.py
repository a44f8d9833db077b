"""Multi-head latent attention ops: latent cache write and attention over the latent cache.

CUDA path: ``csrc/kernels/mla.cu``. CPU path / oracle: plain fp32 PyTorch of the same math.
Reference parity: MlaKvCompress / MlaQAbsorb / MlaAttention
(src/arch/auto_graph_fragments/build_graph.inc.rs:1486-1578).
"""
from __future__ import annotations

import torch

from . import _native as nv
from ._native import F, I, L, P

nv.register("gllm_mla_latent_write", I, [P, L, I, I, I, P, F, P, P, P, P, I, P, I, P])
nv.register("gllm_mla_attention", I, [P, P, P, I, P, I, P, P, P, P, I, I, I, I, F, I, P])
nv.register("gllm_mla_decode_scratch_floats", L, [I, I, I])
nv.register("gllm_mla_decode", I, [P, P, P, I, P, I, P, I, I, I, F, I, P, L, P])

PAGE = 16


def rope_half(x, cos, sin):
    """x [..., d] half-split rotation with cos/sin [..., d/2]."""
    h = x.shape[-1] // 2
    x0, x1 = x[..., :h], x[..., h:]
    return torch.cat([x0 * cos - x1 * sin, x1 * cos + x0 * sin], -1)


def latent_write(kv_a, d_c, norm_w, eps, positions, slot_mapping, cos_t, sin_t, cache):
    """kv_a [T, d_c + d_r] -> cache[page, slot] = [RMSNorm(c_kv) * w | RoPE(k_pe)]."""
    T = kv_a.shape[0]
    d_r = kv_a.shape[1] - d_c
    if not kv_a.is_cuda:
        c = kv_a[:, :d_c].float()
        c = c * torch.rsqrt(c.pow(2).mean(-1, keepdim=True) + eps) * norm_w.float()
        pos = positions.long().clamp(0, cos_t.shape[0] - 1)
        kpe = rope_half(kv_a[:, d_c:].float(), cos_t[pos], sin_t[pos])
        row = torch.cat([c, kpe], -1).to(cache.dtype)
        ok = slot_mapping >= 0
        sl = slot_mapping[ok].long()
        cache.view(-1, d_c + d_r)[sl] = row[ok]
        return
    rc = nv.lib().gllm_mla_latent_write(kv_a.data_ptr(), kv_a.stride(0), T, d_c, d_r, norm_w.data_ptr(), float(eps),
                                        positions.data_ptr(), slot_mapping.data_ptr(), cos_t.data_ptr(),
                                        sin_t.data_ptr(), cos_t.shape[0], cache.data_ptr(), cache.shape[0],
                                        nv.stream_ptr())
    nv.check(rc, "mla_latent_write")


def latent_attention_ref(q, cache, block_tables, q_start, q_len, ctx_lens, n_heads, d_v, scale, causal=True):
    d_k = cache.shape[-1]
    out = torch.zeros((q.shape[0], n_heads * d_v), dtype=q.dtype, device=q.device)
    for s in range(len(q_len)):
        ql, ctx, st = int(q_len[s]), int(ctx_lens[s]), int(q_start[s])
        if ql <= 0 or ctx <= 0:
            continue
        nb = (ctx + PAGE - 1) // PAGE
        rows = cache[block_tables[s, :nb].long()].reshape(-1, d_k)[:ctx].float()
        qs = q[st:st + ql].float().reshape(ql, n_heads, d_k)
        sc = torch.einsum("qhd,kd->hqk", qs, rows) * scale
        if causal:
            pq = torch.arange(ctx - ql, ctx, device=q.device)[:, None]
            pk = torch.arange(ctx, device=q.device)[None, :]
            sc = sc.masked_fill(~(pk <= pq)[None], float("-inf"))
        o = torch.einsum("hqk,kd->qhd", torch.softmax(sc, -1), rows[:, :d_v])
        out[st:st + ql] = o.reshape(ql, n_heads * d_v).to(q.dtype)
    return out


def latent_attention(q, cache, block_tables, q_start, q_len, ctx_lens, row_seq, *, n_heads, d_v, scale, causal=True,
                     out=None):
    """q [T, n_heads * d_k] with rows [q_abs | q_pe]; cache [pages, 16, d_k]; returns [T, n_heads * d_v]."""
    if not q.is_cuda:
        r = latent_attention_ref(q, cache, block_tables, q_start, q_len, ctx_lens, n_heads, d_v, scale, causal)
        if out is not None:
            out.copy_(r)
            return out
        return r
    T = q.shape[0]
    d_k = cache.shape[-1]
    if out is None:
        out = torch.empty((T, n_heads * d_v), dtype=q.dtype, device=q.device)
    rc = nv.lib().gllm_mla_attention(q.data_ptr(), out.data_ptr(), cache.data_ptr(), cache.shape[0],
                                     block_tables.data_ptr(), block_tables.shape[1], row_seq.data_ptr(),
                                     q_start.data_ptr(), q_len.data_ptr(), ctx_lens.data_ptr(), T, n_heads, d_k, d_v,
                                     float(scale), 1 if causal else 0, nv.stream_ptr())
    nv.check(rc, "mla_attention")
    return out


_decode_scratch = {}


def latent_decode(q, cache, block_tables, ctx_lens, *, n_heads, scale, max_ctx=4096, splits=0, out=None):
    """Decode step (one query row per sequence) of the absorbed attention on tensor cores
    (``csrc/kernels/mla_decode.cu``): q [B, n_heads * 576], cache [pages, 16, 576] -> [B, n_heads * 512].
    Needs the DeepSeek geometry (d_c 512, rope 64); other shapes take ``latent_attention``."""
    B = q.shape[0]
    d_k = cache.shape[-1]
    if not q.is_cuda or d_k != 576:
        idx = torch.arange(B, dtype=torch.int32, device=q.device)
        return latent_attention(q, cache, block_tables, idx, torch.ones_like(idx), ctx_lens, idx, n_heads=n_heads, d_v=d_k - 64,
                                scale=scale, out=out)
    if out is None:
        out = torch.empty((B, n_heads * 512), dtype=q.dtype, device=q.device)
    if splits <= 0 and B * ((n_heads + 15) // 16) >= 2 * int(nv.lib().gllm_sm_count()):
        splits = 1          # the rows alone fill the GPU: no KV split, no scratch
    need = int(nv.lib().gllm_mla_decode_scratch_floats(B, n_heads, 16 if splits <= 0 else splits))
    key = (q.device.index, need)
    sc = _decode_scratch.get(key)
    if sc is None:
        sc = _decode_scratch[key] = torch.empty(max(need, 1), dtype=torch.float32, device=q.device)
    rc = nv.lib().gllm_mla_decode(q.data_ptr(), out.data_ptr(), cache.data_ptr(), cache.shape[0], block_tables.data_ptr(),
                                  block_tables.shape[1], ctx_lens.data_ptr(), B, n_heads, int(max_ctx), float(scale), int(splits),
                                  sc.data_ptr(), sc.numel(), nv.stream_ptr())
    nv.check(rc, "mla_decode")
    return out


def latent_prefill(q, cache, block_tables, row_seq, positions, ctx_lens, *, n_heads, scale, causal=True, max_ctx=4096,
                   out=None):
    """Prefill rows of the absorbed attention on the tensor-core kernel of ``latent_decode``: every query row runs as
    a one-token sequence whose context ends at its own position (causal) or at its sequence's end, over its
    sequence's pages. The 16 heads of a tile still share every latent row they read; rows of one sequence re-read the
    same pages, which stay in L2 (a 4 k-token prompt's latent rows are 4.7 MB). q [T, n_heads * 576] ->
    [T, n_heads * 512]. ``row_seq`` [T] maps rows to sequences, ``positions`` [T] are the rows' absolute positions.
    Reference parity: MlaAttention over the latent cache
    (src/arch/auto_graph_fragments/build_graph.inc.rs:1527-1578)."""
    tables = block_tables.index_select(0, row_seq.long())
    if causal:
        row_ctx = (positions + 1).to(torch.int32)
    else:
        row_ctx = ctx_lens.index_select(0, row_seq.long()).to(torch.int32)
    return latent_decode(q, cache, tables.contiguous(), row_ctx.contiguous(), n_heads=n_heads, scale=scale,
                         max_ctx=max_ctx, out=out)
