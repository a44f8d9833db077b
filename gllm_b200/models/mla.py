"""Multi-head latent attention block (DeepSeek-V2/V3 style) on the latent paged cache.

Weights (canonical names): ``q_a_proj`` [q_lora, H] + ``q_a_norm`` + ``q_b_proj`` [heads*(nope+rope), q_lora]
(or a plain ``q_proj`` when ``q_lora_rank == 0``), ``kv_a_proj`` [d_c + rope, H], ``kv_a_norm`` [d_c],
``kv_b_proj`` [heads*(nope+v), d_c], ``o_proj`` [H, heads*v].

Decode and prefill both run the absorbed form: ``q_abs[h] = q_nope[h] @ W_UK[h]`` so that every head attends over
the shared latent rows, then ``out[h] = latent_out[h] @ W_UV[h]^T``. The cache holds d_c + rope values per token
instead of 2 * heads * head_dim. Heads are sharded over tensor-parallel ranks (q_b / kv_b column-parallel,
o_proj row-parallel); the latent cache is replicated.

Reference parity: MLA graph ops and weight roles
(src/arch/auto_graph_fragments/build_graph.inc.rs:1486-1578; shard rules src/loader/weight_shard.rs:133-168).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from .. import ops
from ..ops import mla as MLA
from .config import ModelConfig
from .weights import layer_prefix, shard_range


@dataclass
class MlaWeights:
    q_a: Optional[torch.Tensor]        # [q_lora, H]
    q_a_norm: Optional[torch.Tensor]   # fp32 [q_lora]
    q_b: torch.Tensor                  # [heads_local*(nope+rope), q_lora or H]
    kv_a: torch.Tensor                 # [d_c + rope, H]
    kv_a_norm: torch.Tensor            # fp32 [d_c]
    w_uk: torch.Tensor                 # [heads_local, nope, d_c]
    w_uv: torch.Tensor                 # [heads_local, d_c, v]  (already transposed for out = latent @ w_uv)
    n_heads: int


def pack_mla(cfg: ModelConfig, src, i: int, rank: int, world: int, device, dtype) -> MlaWeights:
    p = layer_prefix(i)
    nope, rope_d, v, d_c = cfg.qk_nope_head_dim, cfg.qk_rope_head_dim, cfg.v_head_dim, cfg.kv_lora_rank
    h0, h1 = shard_range(cfg.num_heads, rank, world)
    qd = nope + rope_d
    from ..ops import linear as L
    mv = lambda t: L.pad_rows(t.to(device, dtype), 128).contiguous()     # GEMM weights: rows padded to the tile
    if cfg.q_lora_rank:
        q_a = mv(src.get(p + "q_a_proj"))
        q_a_norm = src.get(p + "q_a_norm").float().to(device).contiguous()
        q_b = mv(src.get(p + "q_b_proj")[h0 * qd:h1 * qd])
    else:
        q_a, q_a_norm = None, None
        q_b = mv(src.get(p + "q_proj")[h0 * qd:h1 * qd])
    kv_b = src.get(p + "kv_b_proj").reshape(cfg.num_heads, nope + v, d_c)[h0:h1]
    return MlaWeights(q_a=q_a, q_a_norm=q_a_norm, q_b=q_b, kv_a=mv(src.get(p + "kv_a_proj")),
                      kv_a_norm=src.get(p + "kv_a_norm").float().to(device).contiguous(),
                      w_uk=kv_b[:, :nope, :].to(device, dtype).contiguous(),
                      w_uv=kv_b[:, nope:, :].transpose(1, 2).to(device, dtype).contiguous(), n_heads=h1 - h0)


def _row_index(batch, T, device):
    """(row_seq, q_start, q_len) describing which sequence each query row belongs to."""
    if batch.is_decode:
        idx = torch.arange(T, dtype=torch.int32, device=device)
        return idx, idx, torch.ones(T, dtype=torch.int32, device=device)
    S = batch.q_len.shape[0]
    row_seq = torch.repeat_interleave(torch.arange(S, dtype=torch.int32, device=device), batch.q_len.long())
    if row_seq.shape[0] < T:   # padding rows (none in practice) attend to nothing harmful
        row_seq = torch.cat([row_seq, row_seq.new_zeros(T - row_seq.shape[0])])
    return row_seq, batch.q_start, batch.q_len


def mla_attention(model, w: MlaWeights, h, batch, cache, out):
    """h [T, H] normalised hidden; cache [pages, 16, d_c + rope]; writes [T, heads_local * v] into ``out``."""
    c = model.cfg
    T = h.shape[0]
    nope, rope_d, v, d_c = c.qk_nope_head_dim, c.qk_rope_head_dim, c.v_head_dim, c.kv_lora_rank
    nh = w.n_heads
    idx_key = ("mla_idx", T, batch.is_decode)
    if batch.is_decode:
        cached = model.__dict__.setdefault("_mla_cache", {})
        if idx_key not in cached:
            cached[idx_key] = _row_index(batch, T, h.device)
        row_seq, q_start, q_len = cached[idx_key]
    else:
        # the same for every layer of this forward: computed once and kept on the batch
        cached = batch.__dict__.setdefault("_mla_rows", {})
        if "idx" not in cached:
            cached["idx"] = _row_index(batch, T, h.device)
        row_seq, q_start, q_len = cached["idx"]
    # queries
    if w.q_a is not None:
        qa = ops.gemm(h, w.q_a, out_dtype=h.dtype, bn=128)[:, :c.q_lora_rank].contiguous()
        qa = ops.rmsnorm(qa, w.q_a_norm, c.rms_norm_eps)
        q = ops.gemm(qa, w.q_b, out_dtype=h.dtype, bn=128)
    else:
        q = ops.gemm(h, w.q_b, out_dtype=h.dtype, bn=128)
    q = q[:, :nh * (nope + rope_d)].reshape(T, nh, nope + rope_d)
    # latent + rope key -> cache
    kv_a = ops.gemm(h, w.kv_a, out_dtype=h.dtype, bn=128)[:, :d_c + rope_d]
    MLA.latent_write(kv_a, d_c, w.kv_a_norm, c.rms_norm_eps, batch.positions, batch.slot_mapping, model.cos, model.sin,
                     cache)
    # absorb W_UK into the query; rotate the rope part
    pos = batch.positions.long().clamp(0, model.cos.shape[0] - 1)
    q_pe = MLA.rope_half(q[..., nope:].float(), model.cos[pos][:, None, :], model.sin[pos][:, None, :]).to(h.dtype)
    q_abs = torch.bmm(q[..., :nope].transpose(0, 1), w.w_uk).transpose(0, 1)          # [T, nh, d_c]
    q_full = torch.cat([q_abs, q_pe], -1).reshape(T, nh * (d_c + rope_d)).contiguous()
    if batch.is_decode and h.is_cuda and d_c == 512 and rope_d == 64:
        lat = MLA.latent_decode(q_full, cache, batch.block_tables, batch.ctx_lens, n_heads=nh, scale=model.scale,
                                max_ctx=model.max_positions)
    elif h.is_cuda and d_c == 512 and rope_d == 64:
        # prefill chunks on the same tensor-core kernel: one row = one query token over its sequence's pages
        rows = batch.__dict__.setdefault("_mla_rows", {})
        if "tables" not in rows:       # per-row block tables and context lengths: once per forward, not once per layer
            rows["tables"] = batch.block_tables.index_select(0, row_seq.long()).contiguous()
            rows["ctx"] = ((batch.positions + 1) if (batch.causal and c.causal) else
                           batch.ctx_lens.index_select(0, row_seq.long())).to(torch.int32).contiguous()
        lat = MLA.latent_decode(q_full, cache, rows["tables"], rows["ctx"], n_heads=nh, scale=model.scale,
                                max_ctx=model.max_positions)
    else:
        lat = MLA.latent_attention(q_full, cache, batch.block_tables, q_start, q_len, batch.ctx_lens, row_seq, n_heads=nh,
                                   d_v=d_c, scale=model.scale, causal=batch.causal and c.causal)
    o = torch.bmm(lat.reshape(T, nh, d_c).transpose(0, 1), w.w_uv).transpose(0, 1)     # [T, nh, v]
    out[:, :nh * v].copy_(o.reshape(T, nh * v))
    return out[:, :nh * v]


def mla_attention_naive(cfg: ModelConfig, src, i: int, h, positions, cos, sin, scale):
    """Un-absorbed fp32 reference over one full sequence (prefill from position 0): expands K and V per head
    from the latent, standard causal softmax attention. Returns [T, heads * v]."""
    p = layer_prefix(i)
    nope, rope_d, v, d_c, nh = cfg.qk_nope_head_dim, cfg.qk_rope_head_dim, cfg.v_head_dim, cfg.kv_lora_rank, cfg.num_heads
    T = h.shape[0]
    f = lambda n: src.get(p + n).float()
    hf = h.float()
    if cfg.q_lora_rank:
        qa = hf @ f("q_a_proj").t()
        qa = qa * torch.rsqrt(qa.pow(2).mean(-1, keepdim=True) + cfg.rms_norm_eps) * f("q_a_norm")
        q = qa @ f("q_b_proj").t()
    else:
        q = hf @ f("q_proj").t()
    q = q.reshape(T, nh, nope + rope_d)
    kv_a = hf @ f("kv_a_proj").t()
    ckv = kv_a[:, :d_c]
    ckv = ckv * torch.rsqrt(ckv.pow(2).mean(-1, keepdim=True) + cfg.rms_norm_eps) * f("kv_a_norm")
    pos = positions.long()
    k_pe = MLA.rope_half(kv_a[:, d_c:], cos[pos], sin[pos])
    q_pe = MLA.rope_half(q[..., nope:], cos[pos][:, None, :], sin[pos][:, None, :])
    kvb = f("kv_b_proj").reshape(nh, nope + v, d_c)
    k_nope = torch.einsum("tc,hnc->thn", ckv, kvb[:, :nope])
    val = torch.einsum("tc,hvc->thv", ckv, kvb[:, nope:])
    sc = (torch.einsum("qhn,khn->hqk", q[..., :nope], k_nope) + torch.einsum("qhr,kr->hqk", q_pe, k_pe)) * scale
    mask = torch.ones(T, T, dtype=torch.bool).tril()
    sc = sc.masked_fill(~mask[None], float("-inf"))
    o = torch.einsum("hqk,khv->qhv", torch.softmax(sc, -1), val)
    return o.reshape(T, nh * v)
