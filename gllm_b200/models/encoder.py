"""Encoder models (BERT / XLM-R / bge / e5 style, post-LayerNorm, absolute positions) for embeddings,
cross-encoder reranking and classification, plus the pooling / head logic shared with decoder-based variants.

Reference parity: encode path ``embed(+pos/type embeds, LayerNorm) -> bidirectional layers -> MeanPool``
(src/engine/executor_api.rs:633-642, build_graph.inc.rs:2421-2431), cross-encoder head
``CLS -> dense -> tanh -> out_proj(+bias)`` and classifier head (build_graph.inc.rs:2433-2567).
Unlike the reference (one input per call, client_impl.inc.rs:1286-1309), a whole batch of texts runs as one
flat varlen forward.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from .. import ops
from .config import ModelConfig


class EncoderModel:
    def __init__(self, cfg: ModelConfig, src, *, device="cpu", dtype=torch.bfloat16):
        self.cfg, self.device, self.dtype = cfg, torch.device(device), dtype
        g = lambda n, f32=False: src.get(n).to(self.device, torch.float32 if f32 else dtype).contiguous()
        opt = lambda n, f32=False: g(n, f32) if src.has(n) else None
        self.embed = g("embed_tokens")
        self.pos_embed = opt("position_embeddings")
        self.type_embed = opt("token_type_embeddings")
        self.embed_norm_w, self.embed_norm_b = opt("embed_norm", True), opt("embed_norm_bias", True)
        self.layers = []
        D = cfg.head_dim
        for i in range(cfg.num_layers):
            p = f"L{i}."
            wqkv = torch.cat([g(p + "q_proj"), g(p + "k_proj"), g(p + "v_proj")], 0).contiguous()
            bqkv = None
            if src.has(p + "q_proj_bias"):
                bqkv = torch.cat([g(p + "q_proj_bias", True), g(p + "k_proj_bias", True), g(p + "v_proj_bias", True)]).contiguous()
            self.layers.append(dict(
                wqkv=wqkv, bqkv=bqkv, wo=g(p + "o_proj"), bo=opt(p + "o_proj_bias", True),
                ln1_w=opt(p + "post_attn_norm", True), ln1_b=opt(p + "post_attn_norm_bias", True),
                w_up=g(p + "up_proj"), b_up=opt(p + "up_proj_bias", True), w_down=g(p + "down_proj"),
                b_down=opt(p + "down_proj_bias", True), ln2_w=opt(p + "post_ffn_norm", True),
                ln2_b=opt(p + "post_ffn_norm_bias", True)))
        self.pooler_w, self.pooler_b = opt("pooler"), opt("pooler_bias", True)
        self.cls_w, self.cls_b = opt("classifier"), opt("classifier_bias", True)
        self.scale = cfg.attention_scale()

    # ------------------------------------------------------------------------------------------
    def _linear(self, x, w, b):
        N = w.shape[0]
        if x.is_cuda and N % 32 == 0 and x.shape[1] % 8 == 0:
            return ops.gemm(x, w, out_dtype=self.dtype, bias=b, bn=128)
        y = x.float() @ w.float().t()
        if b is not None:
            y = y + b
        return y.to(self.dtype)

    def encode(self, seqs: List[List[int]], token_types: Optional[List[List[int]]] = None) -> torch.Tensor:
        """Token ids of a batch -> final hidden states [T, H] plus (start, len) tensors for pooling."""
        c, dev = self.cfg, self.device
        lens = [len(s) for s in seqs]
        T = sum(lens)
        ids = torch.tensor([t for s in seqs for t in s], dtype=torch.long, device=dev)
        pos = torch.cat([torch.arange(n, device=dev) for n in lens])
        if c.arch in ("xlm-roberta", "roberta") or c.extra.get("position_offset"):
            pos = pos + int(c.extra.get("position_offset", c.pad_token_id + 1))
        x = self.embed[ids].float()
        if self.pos_embed is not None:
            x = x + self.pos_embed[pos].float()
        if self.type_embed is not None:
            tt = torch.zeros(T, dtype=torch.long, device=dev) if token_types is None else \
                torch.tensor([t for s in token_types for t in s], dtype=torch.long, device=dev)
            x = x + self.type_embed[tt].float()
        x = x.to(self.dtype)
        if self.embed_norm_w is not None:
            x = ops.layernorm(x, self.embed_norm_w, self.embed_norm_b, c.layer_norm_eps)
        # attention runs on the paged kernels over a scratch page pool (bidirectional)
        starts = torch.tensor([sum(lens[:i]) for i in range(len(lens))], dtype=torch.int32, device=dev)
        qlen = torch.tensor(lens, dtype=torch.int32, device=dev)
        pages_per = [(n + 15) // 16 for n in lens]
        max_blocks = max(pages_per)
        bt = torch.zeros((len(lens), max_blocks), dtype=torch.int32, device=dev)
        slot = torch.empty(T, dtype=torch.int32, device=dev)
        page0 = 0
        for i, n in enumerate(lens):
            bt[i, :pages_per[i]] = torch.arange(page0, page0 + pages_per[i], dtype=torch.int32, device=dev)
            slot[int(starts[i]):int(starts[i]) + n] = page0 * 16 + torch.arange(n, dtype=torch.int32, device=dev)
            page0 += pages_per[i]
        kv = torch.zeros((page0, 2, c.num_kv_heads, 16, c.head_dim), dtype=self.dtype, device=dev)
        q = torch.empty((T, c.num_heads * c.head_dim), dtype=self.dtype, device=dev)
        pos32 = pos.to(torch.int32)
        for lw in self.layers:
            qkv = self._linear(x, lw["wqkv"], lw["bqkv"])
            ops.rope_kv_write(qkv, n_q=c.num_heads, n_kv=c.num_kv_heads, head_dim=c.head_dim, rot_dim=0,
                              positions=pos32, slot_mapping=slot, cos_t=None, sin_t=None, q_out=q, kv_cache=kv)
            a = ops.paged_prefill(q, kv, bt, starts, qlen, qlen, max_q_len=max(lens), n_q=c.num_heads,
                                  n_kv=c.num_kv_heads, scale=self.scale, causal=False)
            o = self._linear(a, lw["wo"], lw["bo"])
            x = ops.layernorm(o, lw["ln1_w"], lw["ln1_b"], c.layer_norm_eps, residual=x)
            h = self._linear(x, lw["w_up"], lw["b_up"])
            h = torch.nn.functional.gelu(h.float(), approximate="tanh" if "new" in c.hidden_act or "tanh" in c.hidden_act
                                         else "none").to(self.dtype)
            d = self._linear(h, lw["w_down"], lw["b_down"])
            x = ops.layernorm(d, lw["ln2_w"], lw["ln2_b"], c.layer_norm_eps, residual=x)
        return x, starts, qlen

    def embed_batch(self, seqs, pooling: Optional[str] = None) -> torch.Tensor:
        x, starts, qlen = self.encode(seqs)
        return ops.pool(x, starts, qlen, pooling or self.cfg.pooling)

    def score_batch(self, seqs, token_types=None) -> torch.Tensor:
        """Cross-encoder / classifier logits [S, num_labels]: CLS -> (dense -> tanh) -> classifier."""
        x, starts, qlen = self.encode(seqs, token_types)
        cls = ops.pool(x, starts, qlen, "cls")
        if self.pooler_w is not None:
            cls = torch.tanh(cls @ self.pooler_w.float().t() + (self.pooler_b if self.pooler_b is not None else 0))
        if self.cls_w is None:
            raise ValueError("model has no classifier head")
        return cls @ self.cls_w.float().t() + (self.cls_b if self.cls_b is not None else 0)
