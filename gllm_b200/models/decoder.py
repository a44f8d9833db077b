"""Config-driven decoder (Llama / Qwen2 / Qwen3 / Mistral / Gemma-style dense, Qwen3-MoE, and the
DeepSeek MLA variants through ``models/mla.py``) that only calls ops.

Per layer the reference's graph is: input norm -> q/k/v -> head norm -> RoPE -> attention(kv write) ->
o_proj -> residual -> post-attn norm -> gate/up -> SwiGLU -> down -> residual
(src/arch/auto_graph_fragments/build_graph.inc.rs:1445-2045). On B200 that becomes five launches:

    fused QKV GEMM   [RMSNorm as row scale] -> per-head norm -> RoPE -> q buffer + paged KV write
    paged attention  (flash-decode or chunked prefill)
    o_proj GEMM      + residual, leaves the next norm's row statistics behind
    gate/up GEMM     [RMSNorm as row scale] -> SwiGLU epilogue
    down GEMM        + residual, row statistics for the next layer

Architectures the fused kernels do not cover (head_dim != 128, partial rotary, LayerNorm, ...) take the
unfused path built from the same op library. CPU tensors run every op's fp32 oracle, so the same class is
the CPU reference model.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

import torch

from .. import ops
from ..engine.batch import ForwardBatch
from ..ops import linear as L
from . import rope
from .config import ModelConfig
from .weights import DenseLayerWeights, can_fuse, layer_prefix, pack_dense_layer, shard_range, shard_tensor, _fold


class Workspace:
    """Static activation buffers (needed for CUDA-graph replay; also avoids allocator traffic)."""

    def __init__(self, model: "DecoderModel", max_tokens: int):
        c, dev, dt = model.cfg, model.device, model.dtype
        T = max_tokens
        self.max_tokens = T
        H = c.hidden_size
        # With the push form of the fused tensor-parallel all-reduce the row owner stores finished rows into every
        # rank's residual stream, so `x` and the norm statistics live inside the symmetric region of the TP context.
        sym = model.tp.workspace_buffers(T) if (model.tp is not None and hasattr(model.tp, "workspace_buffers")) else None
        self.symmetric = sym is not None
        self.x = sym["x"] if sym else torch.zeros((T, H), dtype=dt, device=dev)
        self.h = torch.zeros((T, H), dtype=dt, device=dev)
        self.q = torch.zeros((T, model.attn_width), dtype=dt, device=dev)
        self.attn = torch.zeros((T, model.attn_width), dtype=dt, device=dev)
        self.qkv = None if (model.fused or c.is_mla) else torch.zeros(
            (T, (model.n_q_local + 2 * model.n_kv_local) * c.head_dim), dtype=dt, device=dev)
        inter = max(model.inter_local, 1)
        self.act = torch.zeros((T, inter), dtype=dt, device=dev)
        self.gu = None if model.fused else torch.zeros((T, 2 * inter), dtype=dt, device=dev)
        self.parts = max(1, (H + 127) // 128)     # room for the narrowest tile width of the residual GEMMs
        self.ss0 = torch.zeros((T, 1), dtype=torch.float32, device=dev)
        self.ss_a = sym["ss_a"] if sym else torch.zeros((T, self.parts), dtype=torch.float32, device=dev)
        self.ss_b = sym["ss_b"] if sym else torch.zeros((T, self.parts), dtype=torch.float32, device=dev)
        self.partial = torch.zeros((T, H), dtype=dt, device=dev) if model.tp_size > 1 else None
        if getattr(model, "sequence_parallel", False):
            # sequence parallel: the residual stream lives as row shards (`xs`), `h` receives the gathered rows in front
            # of the column-parallel GEMMs, statistics come per 256 columns from the gather / reduce-scatter kernels
            per = (T + model.tp_size - 1) // model.tp_size
            self.xs = torch.zeros((per, H), dtype=dt, device=dev)
            self.ss_g = torch.zeros((T, H // 256), dtype=torch.float32, device=dev)
            self.ss_s = torch.zeros((per, H // 256), dtype=torch.float32, device=dev)


class DecoderModel:
    def __init__(self, cfg: ModelConfig, src, *, device="cpu", dtype=torch.bfloat16, tp=None, max_positions=None,
                 fused: Optional[bool] = None, layers: Optional[range] = None, weight_quant: Optional[str] = None,
                 quant_group: int = 32, ep=None, kv_dtype=None, kv_scale: float = 1.0, expert_quant: Optional[str] = None,
                 weight_blob: Optional[bool] = None, sequence_parallel: bool = False, expert_slots: Optional[int] = None,
                 cpu_experts: bool = False):
        """``src`` exposes ``get(name)`` / ``has(name)`` over canonical names; ``tp`` is a
        ``parallel.tensor_parallel.TPContext`` (or None); ``layers`` restricts to a pipeline stage.
        ``sequence_parallel``: between the tensor-parallel GEMMs the residual stream stays sharded by rows (each rank
        keeps ceil(T / tp) rows): the row-parallel GEMMs end in a reduce-scatter instead of an all-reduce and the
        column-parallel GEMMs gather their input rows first (dense bf16 layers of the fused path only).
        ``expert_slots``: keep only this many experts of every MoE layer on the device; the stacks live in pinned host
        memory and are paged in per step (``models.moe.PagedExperts``), for models whose experts do not fit;
        ``cpu_experts``: experts that are not resident and received few rows run on the host instead of being fetched."""
        self.cfg, self.device, self.dtype, self.tp = cfg, torch.device(device), dtype, tp
        self.sequence_parallel = bool(sequence_parallel) and tp is not None
        self.tp_rank = tp.rank if tp else 0
        self.tp_size = tp.size if tp else 1
        self.layer_ids = list(layers) if layers is not None else list(range(cfg.num_layers))
        self.first_stage = 0 in self.layer_ids
        self.last_stage = (cfg.num_layers - 1) in self.layer_ids
        self.kv_dtype = kv_dtype or dtype      # torch.float8_e4m3fn: half the cache bytes; value = stored * kv_scale
        self.kv_scale = float(kv_scale)
        if self.kv_dtype == torch.float8_e4m3fn and cfg.head_dim != 128 and fused is None:
            fused = False        # only the head_dim-128 kernels (fused QKV epilogue, TMA attention) have fp8-page variants
        self.weight_quant = weight_quant
        # "mxfp8" / "nvfp4": both GEMM operands block-scaled on the tensor cores (activations quantised on the device
        # before each GEMM), every fused epilogue kept. Other modes: weight-only quantisation through the dequantising GEMM.
        self.bs_fmt = weight_quant if weight_quant in ("mxfp8", "nvfp4") else None
        self.act_tensor_scale = 1.0 / 64.0      # NVFP4 activations: static second-level scale (values up to 42 exact range)
        if weight_quant is not None and self.bs_fmt is None:
            fused = False        # the dequantising GEMM has no epilogue fusions
        if cfg.gemma3n_structure:
            # several residual streams, a low-rank path beside the attention, per-layer embeddings: the layer runs as
            # separate ops around the stream bookkeeping (models/gemma_ops.py)
            if tp is not None and tp.size > 1:
                raise ValueError("the AltUp / LAuReL / PLE layer structure runs on one rank")
            fused = False
        # the fused layer is the CUDA path; block-scaled models also run it on CPU tensors (every fused op has its fp32
        # restatement), so that the CPU model quantises the same activations as the GPU one and can serve as its oracle
        self.fused = (can_fuse(cfg, self.tp_size) if fused is None else fused) and (
            self.device.type == "cuda" or self.bs_fmt is not None or self.sequence_parallel)
        if self.sequence_parallel and (not self.fused or self.bs_fmt is not None or cfg.is_mla or cfg.is_moe or
                                       cfg.hidden_size % 256 != 0):
            raise ValueError("sequence_parallel needs the fused dense bf16 layer (no MLA, MoE or block-scaled weights) and "
                             "a hidden size that is a multiple of 256")
        if cfg.num_heads % self.tp_size or (cfg.num_kv_heads % self.tp_size and cfg.num_kv_heads >= self.tp_size) or (
                cfg.num_kv_heads < self.tp_size and self.tp_size % cfg.num_kv_heads):
            # with fewer KV heads than ranks each KV head is replicated over tp / num_kv_heads ranks (pack_attention)
            raise ValueError(f"heads {cfg.num_heads}/{cfg.num_kv_heads} not divisible by tp={self.tp_size}")
        self.n_q_local = cfg.num_heads // self.tp_size
        self.n_kv_local = max(1, cfg.num_kv_heads // self.tp_size)
        self.attn_width = self.n_q_local * (max(cfg.head_dim, cfg.v_head_dim) if cfg.is_mla else cfg.head_dim)
        self.inter_local = (cfg.moe_intermediate_size if (cfg.is_moe and cfg.first_k_dense == 0) else
                            cfg.intermediate_size // self.tp_size)
        self.max_positions = max_positions or cfg.max_position_embeddings
        self.cos, self.sin = rope.build_tables(cfg, self.max_positions, self.device)
        # dual RoPE (Gemma 3): sliding-window layers rotate with their own base and no long-context scaling
        self.cos_local = self.sin_local = None
        if cfg.rope_local_theta > 0 and cfg.rotary_dim > 0:
            inv, _ = rope.inv_frequencies(cfg.rotary_dim, cfg.rope_local_theta, type(cfg.rope_scaling)(), self.max_positions)
            ang = torch.arange(self.max_positions, dtype=torch.float64)[:, None] * inv[None, :]
            self.cos_local = ang.cos().float().contiguous().to(self.device)
            self.sin_local = ang.sin().float().contiguous().to(self.device)
        self.act_id = L.ACT_IDS.get(cfg.hidden_act, 0)
        self.res_bn = 256 if cfg.hidden_size % 256 == 0 else 128  # tile width of the residual GEMMs
        self.scale = cfg.attention_scale()

        self.embed = (src.get("embed_tokens").to(self.device, dtype).contiguous()
                      if self.first_stage or cfg.tie_word_embeddings else None)
        self.layers: List[DenseLayerWeights] = []
        for i in self.layer_ids:
            lw = pack_dense_layer(cfg, src, i, self.tp_rank, self.tp_size, self.fused)
            if cfg.is_mla:
                from .mla import pack_mla
                lw.mla = pack_mla(cfg, src, i, self.tp_rank, self.tp_size, self.device, dtype)
            # the source may live on the host (checkpoint files): every packed tensor moves to the model's
            # device here; fp32 tensors (norm weights, biases) stay fp32, the rest takes the compute dtype
            for name, val in list(vars(lw).items()):
                if isinstance(val, torch.Tensor):
                    setattr(lw, name, val.to(self.device, None if val.dtype == torch.float32 and (
                        name.endswith("norm") or name.endswith("bias")) else (dtype if val.is_floating_point() else None)).contiguous())
            if cfg.gemma3n_structure:
                self._load_gemma3n_layer(lw, src, i)
            if weight_quant is not None:
                self._quantize_layer(lw, weight_quant, quant_group)
            if cfg.layer_is_moe(i):
                from .moe import pack_moe_layer
                self.ep = ep if ep is not None else getattr(tp, "ep", None)
                lw.moe = pack_moe_layer(cfg, src, i, self.tp_rank, self.tp_size, self.device, dtype,
                                        ep=ep if ep is not None else getattr(tp, "ep", None), fused=self.fused, tp=tp,
                                        expert_quant=expert_quant or self.bs_fmt)
                if expert_slots:
                    from .moe import ExpertPager, PagedExperts
                    if getattr(self, "expert_pager", None) is None:
                        self.expert_pager = ExpertPager(cfg.num_layers, cfg.num_experts)
                    self.expert_pager.add(i, PagedExperts(lw.moe, i, expert_slots, cpu_experts=cpu_experts))
                    lw.moe.paged = self.expert_pager.layers[i]
            self.layers.append(lw)
        self.final_norm = src.get("final_norm").float().to(self.device).contiguous() if self.last_stage else None
        self.altup_proj = self.altup_unproj = []
        self.ple_table = None
        if cfg.gemma3n_structure:
            n_alt = max(cfg.altup_num_inputs, 1)
            self.altup_proj = [src.get(f"altup_proj.{k}").to(self.device, dtype).contiguous() for k in range(n_alt - 1)]
            self.altup_unproj = [src.get(f"altup_unproj.{k}").to(self.device, dtype).contiguous() for k in range(n_alt - 1)]
            if cfg.ple_dim > 0:
                self.ple_table = src.get("ple_table").to(self.device, dtype).contiguous()
        self.lm_head = None
        if not hasattr(self, "ep"):
            self.ep = None
        self.vocab_local = cfg.vocab_size
        self.vocab_start = 0
        if self.last_stage:
            head = src.get("lm_head") if src.has("lm_head") else src.get("embed_tokens")
            a, b = shard_range(cfg.vocab_size, self.tp_rank, self.tp_size)
            self.vocab_start, self.vocab_local = a, b - a
            head = head[a:b].to(self.device, dtype)
            if self.fused:
                head = _fold(head, self.final_norm, cfg.norm_one_plus_w)
            self.lm_head = L.pad_rows(head, 256).contiguous()
        # Multi-token-prediction heads: ``mtp_proj.{d}`` [vocab, hidden] reads the final-normed hidden state and proposes
        # the token d + 1 positions after the one the main head samples (the reference's graph tail:
        # src/arch/auto_graph_fragments/build_graph.inc.rs:2615-2655). Sharded over the vocabulary like lm_head.
        self.mtp_heads: List[torch.Tensor] = []
        self.last_mtp_logits: List[torch.Tensor] = []
        d = 0
        while self.last_stage and src.has(f"mtp_proj.{d}"):
            w = src.get(f"mtp_proj.{d}")[self.vocab_start:self.vocab_start + self.vocab_local].to(self.device, dtype)
            if self.fused:
                w = _fold(w, self.final_norm, cfg.norm_one_plus_w)
            self.mtp_heads.append(L.pad_rows(w, 256).contiguous())
            d += 1
        self._ws: Optional[Workspace] = None
        self.blob = None
        if weight_blob if weight_blob is not None else self.device.type == "cuda":
            self._pack_blob()

    def _load_gemma3n_layer(self, lw, src, i: int):
        """AltUp / LAuReL / per-layer-embedding tensors of layer ``i`` into ``lw.extra`` (fp32: they are small)."""
        from . import gemma_ops as G
        c, p = self.cfg, layer_prefix(i)
        f = lambda name: src.get(p + name).float().to(self.device).contiguous()
        if c.altup_num_inputs > 1:
            lw.extra["altup"] = G.AltUpWeights(router=f("altup_router"), predict=f("altup_predict"), correct=f("altup_correct"),
                                               router_norm=f("altup_router_norm"), out_scale=f("altup_out_scale"))
        if c.laurel_rank > 0:
            lw.extra["laurel"] = G.LaurelWeights(down=f("laurel_down"), up=f("laurel_up"), norm=f("laurel_norm"))
        if c.ple_dim > 0:
            lw.extra["ple_gate"], lw.extra["ple_proj"], lw.extra["ple_norm"] = f("ple_gate"), f("ple_proj"), f("ple_norm")

    def _pack_blob(self):
        """Re-home the packed dense tensors (per-layer projections and norms, embedding, heads) in ONE contiguous,
        256-byte-aligned allocation with an offset table (engine/weight_blob.py): one upload / one mapping for the
        whole stage, constant per-layer strides for homogeneous layers. Skipped when the device cannot hold the
        second copy that exists while the blob is filled."""
        from ..engine.weight_blob import WeightBlob
        tensors = {}
        for li, lw in zip(self.layer_ids, self.layers):
            for name, val in vars(lw).items():
                if isinstance(val, torch.Tensor) and val.numel() > 0:
                    tensors[f"L{li}.{name}"] = val
        for name in ("embed", "lm_head", "final_norm"):
            val = getattr(self, name, None)
            if isinstance(val, torch.Tensor) and val.numel() > 0:
                tensors[name] = val
        for d, w in enumerate(self.mtp_heads):
            tensors[f"mtp_head.{d}"] = w
        need = sum((t.numel() * t.element_size() + 255) // 256 * 256 for t in tensors.values())
        if self.device.type == "cuda":
            free, _ = torch.cuda.mem_get_info(self.device)
            if need + (1 << 30) > free:
                return
        blob = WeightBlob.pack(tensors, device=self.device)
        for li, lw in zip(self.layer_ids, self.layers):
            for name, val in list(vars(lw).items()):
                if f"L{li}.{name}" in blob.entries:
                    setattr(lw, name, blob.view(f"L{li}.{name}"))
        for name in ("embed", "lm_head", "final_norm"):
            if name in blob.entries:
                setattr(self, name, blob.view(name))
        self.mtp_heads = [blob.view(f"mtp_head.{d}") for d in range(len(self.mtp_heads))]
        self.blob = blob

    # ------------------------------------------------------------------------------------------
    def _quantize_layer(self, lw, mode: str, group: int):
        """Load-time quantisation of the dense projections of one layer into the canonical quantised form (a
        checkpoint that is already quantised arrives here as ``QuantWeight`` and is left alone)."""
        from ..ops.quant_gemm import QuantWeight, quantize
        if self.bs_fmt is not None:
            from ..ops import blockscale as B
            mult = 128 if self.bs_fmt == "mxfp8" else 256
            for name in ("wqkv", "wo", "w_gate_up", "w_down"):
                w = getattr(lw, name, None)
                if isinstance(w, torch.Tensor) and w.dim() == 2 and w.shape[0] > 0:
                    if w.shape[1] % mult:
                        raise ValueError(f"{name}: K = {w.shape[1]} must be a multiple of {mult} for {self.bs_fmt}")
                    setattr(lw, name, B.quantize(w.float(), self.bs_fmt))
            return
        for name in ("wqkv", "wo", "w_gate_up", "w_down"):
            w = getattr(lw, name, None)
            if isinstance(w, torch.Tensor) and w.dim() == 2 and w.shape[0] > 0 and w.shape[1] % 64 == 0 and w.shape[1] % group == 0 \
                    and w.shape[0] % 8 == 0:
                setattr(lw, name, quantize(w.float().cpu(), mode, group).to(self.device))

    def weight_bytes(self) -> int:
        from ..ops.blockscale import BlockScaled
        from ..ops.quant_gemm import QuantWeight
        total = 0
        for lw in self.layers:
            for v in vars(lw).values():
                if isinstance(v, (QuantWeight, BlockScaled)):
                    total += v.nbytes()
                elif isinstance(v, torch.Tensor):
                    total += v.numel() * v.element_size()
        return total

    def kv_cache_shape(self, num_pages: int):
        if self.cfg.is_mla:   # one latent row per token, shared by all heads (and replicated over TP ranks)
            return (num_pages, 16, self.cfg.kv_lora_rank + self.cfg.qk_rope_head_dim)
        return (num_pages, 2, self.n_kv_local, 16, self.cfg.head_dim)

    def alloc_kv_cache(self, num_pages: int) -> List[torch.Tensor]:
        """One cache per layer of this stage; a shared-KV layer's entry is its donor's tensor (no memory of its own)."""
        def one():
            if self.kv_dtype == torch.float8_e4m3fn:
                return torch.zeros(self.kv_cache_shape(num_pages), dtype=torch.uint8, device=self.device).view(torch.float8_e4m3fn)
            return torch.zeros(self.kv_cache_shape(num_pages), dtype=self.dtype, device=self.device)
        caches: List[torch.Tensor] = []
        for li, lw in zip(self.layer_ids, self.layers):
            donor = getattr(lw, "kv_donor", None)
            caches.append(caches[donor - self.layer_ids[0]] if donor is not None else one())
        return caches

    def workspace(self, tokens: int) -> Workspace:
        if self._ws is None or self._ws.max_tokens < tokens:
            self._ws = Workspace(self, max(tokens, 256))
        return self._ws

    # ------------------------------------------------------------------------------------------
    def _rope(self, layer: int):
        """(cos, sin) tables of a layer: the local tables on sliding-window layers of a dual-RoPE model."""
        if self.cos_local is not None and self.cfg.layer_window(layer) > 0:
            return self.cos_local, self.sin_local
        return self.cos, self.sin

    def _attention(self, q, kv, batch: ForwardBatch, out, layer: int, decode_ws):
        window = self.cfg.layer_window(layer)
        cp = getattr(batch, "cp", None)
        if cp is not None and self.layers[layer - self.layer_ids[0]].kv_donor is None:
            # context-parallel prefill: the other ranks' shards of this layer's K/V arrive before the attention
            cp.exchange(kv)
        if batch.is_decode:
            return ops.paged_decode(q, kv, batch.block_tables, batch.ctx_lens, n_q=self.n_q_local, n_kv=self.n_kv_local,
                                    scale=self.scale, out=out, workspace=decode_ws, window=window,
                                    pages_per_split=getattr(decode_ws, "pages_per_split", 32), kv_scale=self.kv_scale)
        return ops.paged_prefill(q, kv, batch.block_tables, batch.q_start, batch.q_len, batch.ctx_lens,
                                 max_q_len=batch.max_q_len, n_q=self.n_q_local, n_kv=self.n_kv_local, scale=self.scale,
                                 out=out, causal=batch.causal and self.cfg.causal, window=window, kv_scale=self.kv_scale)

    def _act_q(self, a, T):
        """Block-scaled copy of the activations ``a`` [T, K] (one reusable buffer per K)."""
        from ..ops import blockscale as B
        if not a.is_cuda:
            return B.quantize_act(a, self.bs_fmt, tensor_scale=self.act_tensor_scale)
        bufs = self.__dict__.setdefault("_actq", {})
        K = a.shape[1]
        buf = bufs.get(K)
        if buf is None or buf.codes.shape[0] < T:
            buf = bufs[K] = B.alloc_act(max(T, self._ws.max_tokens if self._ws else T), K, self.bs_fmt, self.device)
        return B.quantize_act(a, self.bs_fmt, out=buf, tensor_scale=self.act_tensor_scale)

    def _row_parallel_bs(self, a, w, x, ss_out, T):
        """Row-parallel projection on block-scaled operands: x <- a @ w.T + x with the next norm's statistics."""
        from ..ops import blockscale as B
        N = w.rows
        aq = self._act_q(a, T)
        if self.tp_size == 1:
            bn = 128 if T <= 1024 else self.res_bn
            parts = (N + bn - 1) // bn
            ss = ss_out.reshape(-1)[:T * parts].view(T, parts)
            B.gemm_residual(aq, w, x, out=x, row_ss_out=ss, bn=bn)
            return ss
        if aq.codes.is_cuda and hasattr(self.tp, "can_fuse_blockscaled") and self.tp.can_fuse_blockscaled(T, N):
            # tensor parallel: the all-reduce runs in the GEMM's epilogue (low-latency form)
            return self.tp.gemm_allreduce_residual_bs(aq, w, x, ss_out)
        # tensor parallel without the fused form: partial products on the tensor cores, the sum over ranks on NCCL
        import torch.distributed as dist
        p = self._ws.partial[:T]
        B.gemm(aq, w, out=p, bn=128 if T <= 1024 else 256)
        dist.all_reduce(p, group=self.tp.group)
        ss = ss_out.reshape(-1)[:T].view(T, 1)
        ops.rmsnorm(p, None, 0.0, residual=x, h_out=x, ss_out=ss, want_y=False)
        return ss

    def _row_parallel(self, a, w, x, ss_out, T):
        """x <- a @ w.T + x, row statistics into ss_out. With TP the partial sums are all-reduced."""
        if self.bs_fmt is not None and not isinstance(w, torch.Tensor):
            return self._row_parallel_bs(a, w, x, ss_out, T)
        N = w.shape[0]
        bn = self.res_bn
        if self.tp_size == 1 and T <= 256 and N % 128 == 0:
            # decode: 128-wide tiles give twice the tiles and take the split-K path that parks partials in shared
            # memory (measured at M=256: o_proj 24 us vs 39 us, down 40 us vs 51 us with 256-wide tiles)
            bn = 128
        parts = (N + bn - 1) // bn
        ss = ss_out.reshape(-1)[:T * parts].view(T, parts)
        if self.tp_size == 1:
            ops.gemm_residual(a, w, x, out=x, row_ss_out=ss, bn=bn)
            return ss
        return self.tp.gemm_allreduce_residual(a, w, x, ss, self._ws.partial[:T], bn=bn)

    def forward(self, batch: ForwardBatch, kv_caches: List[torch.Tensor], *, hidden_in=None, decode_ws=None,
                return_hidden: bool = False, capture_layers=None, callbacks=None):
        """Returns fp32 logits [R, vocab_local_padded] on the last pipeline stage, else the hidden states.
        ``callbacks``: an ``engine.callbacks.CallbackChain`` run on the residual stream before / after the layers it
        names (eager forward only, never inside a captured graph): a callback may replace the hidden states (RAG or
        knowledge injection, layer skipping), end the layer loop early, or veto; what happened is left in
        ``self.callback_action`` / ``self.callback_info``."""
        if self.cfg.gemma3n_structure:
            if capture_layers is not None or callbacks is not None or hidden_in is not None:
                raise ValueError("capture_layers / callbacks / hidden_in are not available with the AltUp layer structure")
            return self._forward_gemma3n(batch, kv_caches, decode_ws=decode_ws, return_hidden=return_hidden)
        if self.sequence_parallel:
            if capture_layers is not None or callbacks is not None:
                raise ValueError("capture_layers / callbacks are not available with sequence_parallel (no rank holds "
                                 "whole layers' rows)")
            return self._forward_sp(batch, kv_caches, hidden_in=hidden_in, decode_ws=decode_ws, return_hidden=return_hidden)
        c = self.cfg
        T = batch.num_tokens
        ws = self.workspace(T)
        x = ws.x[:T]
        H = c.hidden_size
        captured = {}
        tm = getattr(self, "op_timer", None)      # utils.tracing.GraphTimer: per-op device time inside a CUDA graph
        mark = tm.mark if tm is not None else (lambda name: None)
        mark("begin")
        if self.first_stage and hidden_in is None:
            ops.embed_gather(batch.token_ids, self.embed, scale=c.embedding_scale, out=x, ss_out=ws.ss0[:T])
        else:      # a later pipeline stage, or input embeddings prepared by the caller (multimodal prompts)
            x.copy_(hidden_in)
            if self.fused:
                ops.rmsnorm(x, None, c.rms_norm_eps, ss_out=ws.ss0[:T], want_y=False)
        ss_in = ws.ss0[:T]
        self.callback_action, self.callback_info = None, {}
        stop = False
        for li, lw in zip(self.layer_ids, self.layers):
            if callbacks is not None:
                ss_in, stop = self._run_callbacks(callbacks, "pre", li, x, ss_in, ws, T)
                if stop:
                    break
            # a shared-KV layer projects queries only (n_kv = 0: no K / V tiles, nothing written) and attends over its
            # donor's pages
            shared = lw.kv_donor is not None
            kv = kv_caches[(lw.kv_donor if shared else li) - self.layer_ids[0]]
            slots = None if shared else batch.slot_mapping
            cos_l, sin_l = self._rope(li)
            if self.fused:
                if self.bs_fmt is not None:
                    from ..ops import blockscale as B
                    B.gemm_qkv(self._act_q(x, T), lw.wqkv, n_q=lw.n_q, n_kv=lw.n_kv, q_out=ws.q[:T], kv_cache=kv,
                               slot_mapping=slots, positions=batch.positions, cos_t=cos_l,
                               sin_t=sin_l, q_norm_w=lw.q_norm, k_norm_w=lw.k_norm, qk_eps=c.qk_norm_eps,
                               row_ss=ss_in, norm_dim=H, eps=c.rms_norm_eps, bias=lw.qkv_bias, kv_scale=self.kv_scale)
                else:
                    ops.gemm_qkv(x, lw.wqkv, n_q=lw.n_q, n_kv=lw.n_kv, q_out=ws.q[:T], kv_cache=kv,
                                 slot_mapping=slots, positions=batch.positions, cos_t=cos_l,
                                 sin_t=sin_l, q_norm_w=lw.q_norm, k_norm_w=lw.k_norm, qk_eps=c.qk_norm_eps,
                                 row_ss=ss_in, norm_dim=H, eps=c.rms_norm_eps, bias=lw.qkv_bias, kv_scale=self.kv_scale)
                mark("qkv_gemm")
                self._attention(ws.q[:T], kv, batch, ws.attn[:T], li, decode_ws)
                mark("attention")
                ss_mid = self._row_parallel(ws.attn[:T], lw.wo, x, ws.ss_b[:T], T)
                mark("o_proj")
                if lw.moe is not None:
                    ss_in = lw.moe.forward(self, x, ss_mid, ws.ss_a[:T], T)
                    mark("moe")
                else:
                    # the packing is tile-width independent: the width recorded with the weight fills one wave of SMs
                    # at decode sizes, prefill chunks take the widest tile (best tensor-core rate)
                    if self.bs_fmt is not None:
                        from ..ops import blockscale as B
                        inter = lw.w_down.k
                        B.gemm_glu(self._act_q(x, T), lw.w_gate_up, act=self.act_id, out=ws.act[:T, :inter], row_ss=ss_mid,
                                   norm_dim=H, eps=c.rms_norm_eps, bn=256 if (T > 1024 and lw.w_gate_up.rows % 256 == 0) else 128)
                        mark("gate_up_gemm")
                        ss_in = self._row_parallel(ws.act[:T, :inter], lw.w_down, x, ws.ss_a[:T], T)
                        mark("down_proj")
                    else:
                        glu_bn = 256 if (T > 1024 and lw.w_gate_up.shape[0] % 256 == 0) else lw.glu_bn
                        ops.gemm_glu(x, lw.w_gate_up, act=self.act_id, out=ws.act[:T, :lw.w_down.shape[1]],
                                     row_ss=ss_mid, norm_dim=H, eps=c.rms_norm_eps, bn=glu_bn)
                        mark("gate_up_gemm")
                        ss_in = self._row_parallel(ws.act[:T, :lw.w_down.shape[1]], lw.w_down, x, ws.ss_a[:T], T)
                        mark("down_proj")
            else:
                h = ws.h[:T]
                ops.rmsnorm(x, lw.input_norm, c.rms_norm_eps, one_plus_w=c.norm_one_plus_w, out=h)
                if lw.mla is not None:
                    from .mla import mla_attention
                    attn = mla_attention(self, lw.mla, h, batch, kv, ws.attn[:T])
                    self._row_parallel(attn, lw.wo, x, ws.ss_b[:T], T)
                else:
                    qkv = ops.gemm(h, lw.wqkv, out=ws.qkv[:T, :lw.wqkv.shape[0]], out_dtype=self.dtype, bias=lw.qkv_bias, bn=128)
                    ops.rope_kv_write(qkv, n_q=lw.n_q, n_kv=lw.n_kv, head_dim=c.head_dim, rot_dim=c.rotary_dim,
                                      positions=batch.positions, slot_mapping=slots, cos_t=cos_l,
                                      sin_t=sin_l, q_out=ws.q[:T], kv_cache=kv, q_norm_w=lw.q_norm,
                                      k_norm_w=lw.k_norm, qk_eps=c.qk_norm_eps, kv_scale=self.kv_scale)
                    self._attention(ws.q[:T], kv, batch, ws.attn[:T], li, decode_ws)
                    self._row_parallel(ws.attn[:T], lw.wo, x, ws.ss_b[:T], T)
                ops.rmsnorm(x, lw.post_attn_norm, c.rms_norm_eps, one_plus_w=c.norm_one_plus_w, out=h)
                if lw.moe is not None:
                    lw.moe.forward_unfused(self, x, h, T)
                else:
                    gu = ops.gemm(h, lw.w_gate_up, out=ws.gu[:T, :lw.w_gate_up.shape[0]], out_dtype=self.dtype, bn=128)
                    act = ops.glu(gu, self.act_id, out=ws.act[:T, :lw.w_down.shape[1]])
                    self._row_parallel(act, lw.w_down, x, ws.ss_a[:T], T)
            if capture_layers is not None and li in capture_layers:
                captured[li] = x.clone()
            if callbacks is not None:
                ss_in, stop = self._run_callbacks(callbacks, "post", li, x, ss_in, ws, T)
                if stop:
                    break
        if capture_layers is not None:
            self.captured = captured
        if not self.last_stage or return_hidden:
            return x
        rows = batch.logits_rows
        cap = float(c.logit_softcap or 0.0)       # final-logit soft cap: applied in the lm_head GEMM's epilogue
        if self.fused:
            xr, sr = (x, ss_in) if rows is None else (x.index_select(0, rows), ss_in.index_select(0, rows))
            logits = ops.gemm(xr, self.lm_head, out_dtype=torch.float32, row_ss=sr, norm_dim=H, eps=c.rms_norm_eps,
                              bn=256, softcap=cap)
        else:
            xr = x if rows is None else x.index_select(0, rows)
            hn = ops.rmsnorm(xr, self.final_norm, c.rms_norm_eps, one_plus_w=c.norm_one_plus_w)
            logits = ops.gemm(hn, self.lm_head, out_dtype=torch.float32, bn=256, softcap=cap)
        mark("lm_head")
        self.last_mtp_logits = []
        if self.mtp_heads and getattr(batch, "want_mtp", False):
            for w in self.mtp_heads:      # same rows, same norm handling as the main head
                if self.fused:
                    self.last_mtp_logits.append(ops.gemm(xr, w, out_dtype=torch.float32, row_ss=sr, norm_dim=H,
                                                         eps=c.rms_norm_eps, bn=256))
                else:
                    self.last_mtp_logits.append(ops.gemm(hn, w, out_dtype=torch.float32, bn=256))
        return logits

    def _forward_gemma3n(self, batch: ForwardBatch, kv_caches, *, decode_ws=None, return_hidden=False):
        """The Gemma-3n residual structure around the ordinary attention and MLP ops.

        ``altup_num_inputs`` residual streams [n, T, H] (stream 0 is the embedding, the others are projections of it
        rescaled to its magnitude); per layer: AltUp predicts every stream from all of them, the layer runs on the
        ACTIVE stream only (attention with the LAuReL low-rank path beside it, then the MLP), AltUp spreads the
        layer's innovation to all streams, and the layer's slice of the per-layer token embedding, gated by the active
        stream, is added to the other streams. After the last layer the streams are projected back and averaged.
        Reference: AltUpPredict / AltUpCorrect / AltUpInject, LAuReL and the PLE gather in the graph builder
        (src/arch/auto_graph_fragments/build_graph.inc.rs:695, 1064, 1115, 1811-1846)."""
        from . import gemma_ops as G
        c = self.cfg
        T = batch.num_tokens
        ws = self.workspace(T)
        x, h = ws.x[:T], ws.h[:T]
        eps = c.rms_norm_eps
        n, act_i = max(c.altup_num_inputs, 1), c.altup_active_idx
        ops.embed_gather(batch.token_ids, self.embed, scale=c.embedding_scale, out=x, ss_out=ws.ss0[:T])
        x0 = x.clone()
        rms = lambda t: t.float().pow(2).mean(-1, keepdim=True).clamp_min(1e-12).sqrt()
        streams = [x0]
        for w in self.altup_proj:                         # the other streams start as projections at the same magnitude
            p = ops.gemm(x0, w, out_dtype=self.dtype, bn=128)[:, :c.hidden_size].float()
            streams.append((p * rms(x0) / rms(p)).to(self.dtype))
        streams = torch.stack(streams)                    # [n, T, H]
        for li, lw in zip(self.layer_ids, self.layers):
            shared = lw.kv_donor is not None
            kv = kv_caches[(lw.kv_donor if shared else li) - self.layer_ids[0]]
            slots = None if shared else batch.slot_mapping
            aw = lw.extra.get("altup")
            pred = G.altup_predict(streams, aw, act_i, eps) if aw is not None else streams
            x.copy_(pred[act_i])
            ops.rmsnorm(x, lw.input_norm, eps, one_plus_w=c.norm_one_plus_w, out=h)
            qkv = ops.gemm(h, lw.wqkv, out=ws.qkv[:T, :lw.wqkv.shape[0]], out_dtype=self.dtype, bias=lw.qkv_bias, bn=128)
            ops.rope_kv_write(qkv, n_q=lw.n_q, n_kv=lw.n_kv, head_dim=c.head_dim, rot_dim=c.rotary_dim,
                              positions=batch.positions, slot_mapping=slots, cos_t=self._rope(li)[0], sin_t=self._rope(li)[1],
                              q_out=ws.q[:T],
                              kv_cache=kv, q_norm_w=lw.q_norm, k_norm_w=lw.k_norm, qk_eps=c.qk_norm_eps, kv_scale=self.kv_scale)
            self._attention(ws.q[:T], kv, batch, ws.attn[:T], li, decode_ws)
            self._row_parallel(ws.attn[:T], lw.wo, x, ws.ss_b[:T], T)                       # x = stream + attention
            if "laurel" in lw.extra:                      # (x + h + norm(up(down(h)))) / sqrt(2), h the normalised input
                x.copy_(G.laurel(h, x, lw.extra["laurel"], eps))
            ops.rmsnorm(x, lw.post_attn_norm, eps, one_plus_w=c.norm_one_plus_w, out=h)
            gu = ops.gemm(h, lw.w_gate_up, out=ws.gu[:T, :lw.w_gate_up.shape[0]], out_dtype=self.dtype, bn=128)
            a = ops.glu(gu, self.act_id, out=ws.act[:T, :lw.w_down.shape[1]])
            self._row_parallel(a, lw.w_down, x, ws.ss_a[:T], T)
            if aw is None:
                streams = x.clone()[None]
                continue
            corr = G.altup_correct(pred, x, aw, act_i, eps)
            ple = None
            if self.ple_table is not None:
                pe = G.ple_gather(self.ple_table, batch.token_ids, li, c.num_layers)           # [T, d]
                g = L._act_ref(corr[act_i].float() @ lw.extra["ple_gate"].t(), self.act_id) * pe
                ple = g @ lw.extra["ple_proj"].t()
                ple = ple * torch.rsqrt(ple.pow(2).mean(-1, keepdim=True) + eps) * lw.extra["ple_norm"]
            streams = G.altup_inject(corr, ple, aw, act_i)
        out = [streams[0].float()]
        for k, w in enumerate(self.altup_unproj):          # back to the embedding's space and magnitude, then the mean
            u = ops.gemm(streams[k + 1].contiguous(), w, out_dtype=self.dtype, bn=128)[:, :c.hidden_size].float()
            out.append(u * rms(streams[0]) / rms(u))
        x.copy_(torch.stack(out).mean(0).to(self.dtype))
        if not self.last_stage or return_hidden:
            return x
        rows = batch.logits_rows
        xr = x if rows is None else x.index_select(0, rows)
        hn = ops.rmsnorm(xr, self.final_norm, eps, one_plus_w=c.norm_one_plus_w)
        self.last_mtp_logits = []
        return ops.gemm(hn, self.lm_head, out_dtype=torch.float32, bn=256, softcap=float(c.logit_softcap or 0.0))

    def _run_callbacks(self, callbacks, when: str, li: int, x, ss_in, ws, T: int):
        """One port of the callback chain. Returns (row statistics of x for the next fused GEMM, stop the layer loop)."""
        from ..engine.callbacks import CallbackAction
        if li not in callbacks.layers_of_interest(self.cfg.num_layers):
            return ss_in, False
        r = callbacks.run(when, li, x)
        self.callback_info.update(r.info)
        if r.hidden is not None:
            x.copy_(r.hidden.to(x.dtype))
            if self.fused:      # the statistics came from the previous GEMM's epilogue: recompute them for the new rows
                ops.rmsnorm(x, None, self.cfg.rms_norm_eps, ss_out=ws.ss0[:T], want_y=False)
                ss_in = ws.ss0[:T]
        if r.action in (CallbackAction.EXIT_EARLY, CallbackAction.VETO):
            self.callback_action = r.action
            self.callback_info.setdefault("stopped_at", (when, li))
            return ss_in, True
        if r.action == CallbackAction.REPLACE:
            self.callback_action = self.callback_action or r.action
        return ss_in, False

    def _forward_sp(self, batch: ForwardBatch, kv_caches, *, hidden_in=None, decode_ws=None, return_hidden=False):
        """The fused dense layer with the residual stream sharded by rows over the tensor-parallel ranks.

        Per layer: [all-gather rows + QKV GEMM] -> attention -> [o_proj GEMM + reduce-scatter into the row shard]
        -> [all-gather rows + gate/up GEMM] -> [down GEMM + reduce-scatter]. Each bracket is one kernel in the
        low-latency form of the TP context (ordinary collectives otherwise). Against the all-reduce form a rank
        receives (W-1)/W of the rows once per GEMM pair instead of twice, and the norm statistics are computed on the
        gathered rows. The first layer reads the embedding rows, which every rank computes itself. Reference:
        tp_reduce_scatter / tp_column_parallel_all_gather (src/engine/coordinator/compute.rs:148-164, 246-271)."""
        c, tp = self.cfg, self.tp
        T = batch.num_tokens
        ws = self.workspace(T)
        H = c.hidden_size
        x, h, xs, ss_g = ws.x[:T], ws.h[:T], ws.xs, ws.ss_g[:T]
        lo, n_own = tp.shard_rows(T)
        tm = getattr(self, "op_timer", None)
        mark = tm.mark if tm is not None else (lambda name: None)
        mark("begin")
        if self.first_stage and hidden_in is None:
            ops.embed_gather(batch.token_ids, self.embed, scale=c.embedding_scale, out=x, ss_out=ws.ss0[:T])
        else:
            x.copy_(hidden_in)
            ops.rmsnorm(x, None, c.rms_norm_eps, ss_out=ws.ss0[:T], want_y=False)
        if n_own:
            xs[:n_own].copy_(x[lo:lo + n_own])
        a_in, ss_in = x, ws.ss0[:T]
        for idx, (li, lw) in enumerate(zip(self.layer_ids, self.layers)):
            shared = lw.kv_donor is not None
            kv = kv_caches[(lw.kv_donor if shared else li) - self.layer_ids[0]]
            slots = None if shared else batch.slot_mapping
            if idx > 0:
                tp.allgather_input(xs, h, ss_out=ss_g)      # consumed by the QKV GEMM below
                a_in, ss_in = h, ss_g
            ops.gemm_qkv(a_in, lw.wqkv, n_q=lw.n_q, n_kv=lw.n_kv, q_out=ws.q[:T], kv_cache=kv, slot_mapping=slots,
                         positions=batch.positions, cos_t=self._rope(li)[0], sin_t=self._rope(li)[1], q_norm_w=lw.q_norm,
                         k_norm_w=lw.k_norm, qk_eps=c.qk_norm_eps, row_ss=ss_in, norm_dim=H, eps=c.rms_norm_eps,
                         bias=lw.qkv_bias, kv_scale=self.kv_scale)
            mark("qkv_gemm")
            self._attention(ws.q[:T], kv, batch, ws.attn[:T], li, decode_ws)
            mark("attention")
            tp.gemm_reduce_scatter_residual(ws.attn[:T], lw.wo, xs, ws.ss_s, T)
            mark("o_proj")
            tp.allgather_input(xs, h, ss_out=ss_g)          # consumed by the gate/up GEMM below
            inter = lw.w_down.shape[1]
            glu_bn = 256 if (T > 1024 and lw.w_gate_up.shape[0] % 256 == 0) else lw.glu_bn
            ops.gemm_glu(h, lw.w_gate_up, act=self.act_id, out=ws.act[:T, :inter], row_ss=ss_g, norm_dim=H,
                         eps=c.rms_norm_eps, bn=glu_bn)
            mark("gate_up_gemm")
            tp.gemm_reduce_scatter_residual(ws.act[:T, :inter], lw.w_down, xs, ws.ss_s, T)
            mark("down_proj")
        tp.allgather_rows(xs, x, ss_out=ss_g)
        if not self.last_stage or return_hidden:
            return x
        rows = batch.logits_rows
        xr, sr = (x, ss_g) if rows is None else (x.index_select(0, rows), ss_g.index_select(0, rows))
        logits = ops.gemm(xr, self.lm_head, out_dtype=torch.float32, row_ss=sr, norm_dim=H, eps=c.rms_norm_eps, bn=256,
                          softcap=float(c.logit_softcap or 0.0))
        mark("lm_head")
        self.last_mtp_logits = []
        if self.mtp_heads and getattr(batch, "want_mtp", False):
            for w in self.mtp_heads:
                self.last_mtp_logits.append(ops.gemm(xr, w, out_dtype=torch.float32, row_ss=sr, norm_dim=H,
                                                     eps=c.rms_norm_eps, bn=256))
        return logits

    # ------------------------------------------------------------------------------------------
    def head_logits(self, xr):
        """fp32 logits [R, vocab_local_padded] of residual-stream rows ``xr`` (what ``forward(return_hidden=True)``
        returns): final norm + lm_head, with the soft cap; in the fused layout the norm weight lives in the head and
        the rows' statistics are taken here."""
        c = self.cfg
        cap = float(c.logit_softcap or 0.0)
        if self.fused:
            ss = torch.empty((xr.shape[0], 1), dtype=torch.float32, device=xr.device)
            ops.rmsnorm(xr, None, c.rms_norm_eps, ss_out=ss, want_y=False)
            return ops.gemm(xr, self.lm_head, out_dtype=torch.float32, row_ss=ss, norm_dim=c.hidden_size, eps=c.rms_norm_eps,
                            bn=256, softcap=cap)
        hn = ops.rmsnorm(xr, self.final_norm, c.rms_norm_eps, one_plus_w=c.norm_one_plus_w)
        return ops.gemm(hn, self.lm_head, out_dtype=torch.float32, bn=256, softcap=cap)

    def final_hidden(self, x):
        """Final-norm hidden states (embedding / head-routing consumers)."""
        return ops.rmsnorm(x, self.final_norm, self.cfg.rms_norm_eps, one_plus_w=self.cfg.norm_one_plus_w)
