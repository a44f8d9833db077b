"""Canonical weight names, random initialisation of a named architecture, tensor-parallel slicing, and the
weight packer that turns checkpoint tensors into the layouts the sm_100a kernels consume.

Reference parity:
  * canonical names ``embed_tokens``, ``L{n}.q_proj`` ... (src/loader/name_map.rs:7-293)
  * TP shard rules: q/k/v/gate/up/lm_head column-parallel (split out-features), o_proj/down_proj
    row-parallel (split in-features), norms / router replicated (src/loader/weight_shard.rs:133-168)
  * one contiguous, kernel-friendly weight blob per model (src/engine/mega_kernel/pack_observe.inc.rs:116-735);
    here "kernel-friendly" means K-major bf16 tiles for TMA, fused QKV, tile-interleaved gate/up, and the
    RMSNorm weights folded into the following projection.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional

import torch

from ..ops import linear as L
from .config import ModelConfig


def layer_prefix(i: int) -> str:
    return f"L{i}."


# ------------------------------------------------------------------------------------------------
# tensor-parallel slicing (pure functions of rank / world)
# ------------------------------------------------------------------------------------------------
COLUMN_PARALLEL = ("q_proj", "k_proj", "v_proj", "qkv_proj", "gate_proj", "up_proj", "lm_head", "q_b_proj",
                   "kv_b_proj", "k_b_proj", "v_b_proj")
ROW_PARALLEL = ("o_proj", "down_proj")


def shard_kind(name: str) -> str:
    base = name.rsplit(".", 1)[-1]
    if base.endswith("_bias"):
        base = base[:-5]
    if base in COLUMN_PARALLEL:
        return "column"
    if base in ROW_PARALLEL:
        return "row"
    return "replicated"


def shard_range(n: int, rank: int, world: int):
    """Contiguous split with the remainder spread over the first ranks."""
    base, rem = divmod(n, world)
    start = rank * base + min(rank, rem)
    return start, start + base + (1 if rank < rem else 0)


def shard_tensor(name: str, t: torch.Tensor, rank: int, world: int, *, head_dim: int = 0) -> torch.Tensor:
    """Slice ``t`` ([out, in] or [out]) for ``rank``. Head-structured projections split on head
    boundaries (``head_dim`` > 0) so no head is torn between ranks."""
    if world == 1:
        return t
    kind = shard_kind(name)
    if kind == "replicated":
        return t
    is_bias = name.endswith("_bias")
    if kind == "column" or is_bias and kind == "column":
        units = t.shape[0] // head_dim if head_dim else t.shape[0]
        a, b = shard_range(units, rank, world)
        mul = head_dim or 1
        return t[a * mul:b * mul].contiguous()
    if is_bias:  # bias of a row-parallel layer is added once (rank 0)
        return t if rank == 0 else torch.zeros_like(t)
    units = t.shape[1] // head_dim if head_dim else t.shape[1]
    a, b = shard_range(units, rank, world)
    mul = head_dim or 1
    return t[:, a * mul:b * mul].contiguous()


# ------------------------------------------------------------------------------------------------
# random initialisation (seeded normal, std 0.02) of the local shard, generated on the device
# ------------------------------------------------------------------------------------------------
class RandomWeights:
    """Lazily generates canonical tensors of ``cfg``'s architecture. Every tensor has its own seed derived
    from its name, so any rank can materialise exactly its slice of the same global model."""

    def __init__(self, cfg: ModelConfig, device="cpu", dtype=torch.bfloat16, seed=0, std=0.02):
        self.cfg, self.device, self.dtype, self.seed, self.std = cfg, torch.device(device), dtype, seed, std

    def _gen(self, name: str, shape, *, ones=False) -> torch.Tensor:
        if ones:
            g = torch.Generator(device="cpu").manual_seed((hash_name(name) + self.seed) & 0x7FFFFFFF)
            return (1.0 + 0.1 * torch.randn(shape, generator=g)).to(torch.float32).to(self.device)
        g = torch.Generator(device=self.device).manual_seed((hash_name(name) + self.seed) & 0x7FFFFFFF)
        t = torch.empty(shape, dtype=torch.float32 if self.device.type == "cpu" else self.dtype, device=self.device)
        t.normal_(0.0, self.std, generator=g)
        return t.to(self.dtype)

    def shape_of(self, name: str):
        c = self.cfg
        base = name.rsplit(".", 1)[-1]
        H, D = c.hidden_size, c.head_dim
        table = {
            "embed_tokens": (c.vocab_size, H), "lm_head": (c.vocab_size, H), "final_norm": (H,),
            "input_norm": (H,), "post_attn_norm": (H,), "q_norm": (D,), "k_norm": (D,),
            "q_proj": (c.num_heads * D, H), "k_proj": (c.num_kv_heads * D, H), "v_proj": (c.num_kv_heads * D, H),
            "o_proj": (H, c.num_heads * D), "q_proj_bias": (c.num_heads * D,), "k_proj_bias": (c.num_kv_heads * D,),
            "v_proj_bias": (c.num_kv_heads * D,), "router": (c.num_experts, H),
        }
        if c.is_mla:
            table["o_proj"] = (H, c.num_heads * c.v_head_dim)
            table["q_proj"] = (c.num_heads * (c.qk_nope_head_dim + c.qk_rope_head_dim), H)
        if c.norm_type == "layer" or c.kind != "chat":     # encoder checkpoints (BERT / XLM-R style) and their heads
            I = c.intermediate_size
            table.update({
                "position_embeddings": (c.max_position_embeddings, H), "token_type_embeddings": (max(c.type_vocab_size, 1), H),
                "embed_norm": (H,), "embed_norm_bias": (H,), "post_ffn_norm": (H,), "post_attn_norm_bias": (H,),
                "post_ffn_norm_bias": (H,), "o_proj_bias": (H,), "up_proj_bias": (I,), "down_proj_bias": (H,),
                "pooler": (H, H), "pooler_bias": (H,), "classifier": (max(getattr(c, "num_labels", 0) or 1, 1), H),
                "classifier_bias": (max(getattr(c, "num_labels", 0) or 1, 1),)})
        if base in table:
            return table[base]
        n_alt, r_l, d_ple = max(c.altup_num_inputs, 1), max(c.laurel_rank, 1), max(c.ple_dim, 1)
        gemma3n = {"altup_router": (n_alt, H), "altup_predict": (n_alt * n_alt, n_alt), "altup_correct": (n_alt, n_alt),
                   "altup_router_norm": (H,), "altup_out_scale": (H,), "laurel_down": (r_l, H), "laurel_up": (H, r_l),
                   "laurel_norm": (H,), "ple_table": (c.vocab_size, c.num_layers * d_ple), "ple_gate": (d_ple, H),
                   "ple_proj": (H, d_ple), "ple_norm": (H,)}
        if base in gemma3n:
            return gemma3n[base]
        if name.startswith("altup_proj.") or name.startswith("altup_unproj."):
            return (H, H)
        inter = c.intermediate_size
        if ".experts." in name:
            inter = c.moe_intermediate_size
        elif ".shared_expert." in name:
            inter = (c.shared_expert_intermediate_size or c.moe_intermediate_size) * max(c.num_shared_experts, 1)
        if base in ("gate_proj", "up_proj"):
            return (inter, H)
        if base == "down_proj":
            return (H, inter)
        if c.is_mla:
            qd = c.qk_nope_head_dim + c.qk_rope_head_dim
            mla = {"q_a_proj": (c.q_lora_rank, H), "q_a_norm": (c.q_lora_rank,),
                   "q_b_proj": (c.num_heads * qd, c.q_lora_rank),
                   "kv_a_proj": (c.kv_lora_rank + c.qk_rope_head_dim, H), "kv_a_norm": (c.kv_lora_rank,),
                   "kv_b_proj": (c.num_heads * (c.qk_nope_head_dim + c.v_head_dim), c.kv_lora_rank),
                   "o_proj": (H, c.num_heads * c.v_head_dim), "q_proj": (c.num_heads * qd, H)}
            if base in mla:
                return mla[base]
        raise KeyError(name)

    def get(self, name: str) -> torch.Tensor:
        base = name.rsplit(".", 1)[-1]
        shape = self.shape_of(name)
        return self._gen(name, shape, ones=base.endswith("norm") or base == "altup_out_scale")

    def has(self, name: str) -> bool:
        c = self.cfg
        base = name.rsplit(".", 1)[-1]
        if base == "lm_head":
            return not c.tie_word_embeddings
        if base in ("q_norm", "k_norm"):
            return c.qk_norm
        if base in ("classifier", "classifier_bias"):
            return (getattr(c, "num_labels", 0) or 0) > 0
        if base in ("token_type_embeddings",):
            return c.type_vocab_size > 0
        if base in ("up_proj_bias", "down_proj_bias"):
            return bool(getattr(c, "mlp_bias", False))
        if base.endswith("norm_bias"):
            return c.norm_type == "layer"
        if base.endswith("_bias"):
            return c.attention_bias
        try:
            self.shape_of(name)
            return True
        except KeyError:
            return False


def hash_name(name: str) -> int:
    h = 2166136261
    for ch in name.encode():
        h = ((h ^ ch) * 16777619) & 0xFFFFFFFF
    return h


class DictWeights:
    """Weights already in memory under canonical names (what the loaders produce)."""

    def __init__(self, tensors: Dict[str, torch.Tensor], device="cpu", dtype=None):
        self.t, self.device, self.dtype = tensors, torch.device(device), dtype

    def has(self, name: str) -> bool:
        return name in self.t

    def get(self, name: str) -> torch.Tensor:
        t = self.t[name]
        if self.dtype is not None and t.is_floating_point() and not name.rsplit(".", 1)[-1].endswith("norm"):
            t = t.to(self.dtype)
        return t.to(self.device)


# ------------------------------------------------------------------------------------------------
# packed per-layer weights
# ------------------------------------------------------------------------------------------------
@dataclass
class DenseLayerWeights:
    fused: bool
    wqkv: torch.Tensor                       # [(Hq+2Hkv)*D, H]  (input-norm weight folded in when fused)
    qkv_bias: Optional[torch.Tensor]         # fp32
    q_norm: Optional[torch.Tensor]           # fp32 [D]
    k_norm: Optional[torch.Tensor]
    wo: torch.Tensor                         # [H, Hq*D]
    w_gate_up: Optional[torch.Tensor]        # fused: tile-interleaved [2I, H]; unfused: [gate | up] stacked
    w_down: Optional[torch.Tensor]           # [H, I]
    input_norm: torch.Tensor                 # fp32 [H] (used by the unfused path)
    post_attn_norm: torch.Tensor
    glu_bn: int = 256
    n_q: int = 0
    n_kv: int = 0
    moe: Optional[object] = None
    mla: Optional[object] = None
    kv_donor: Optional[int] = None           # shared-KV layer: attends over this earlier layer's cache, writes none
    extra: Dict[str, torch.Tensor] = field(default_factory=dict)


def _fold(w: torch.Tensor, norm_w: torch.Tensor, one_plus: bool) -> torch.Tensor:
    g = (1.0 + norm_w.float()) if one_plus else norm_w.float()
    return (w.float() * g[None, :].to(w.device)).to(w.dtype)


def can_fuse(cfg: ModelConfig, tp: int = 1) -> bool:
    """The fused tcgen05 path needs head_dim 128 with full rotary, RMSNorm, SiLU/GELU-tanh GLU, causal."""
    inter = cfg.intermediate_size // tp
    return (cfg.head_dim == 128 and cfg.norm_type == "rms" and cfg.rotary_dim == 128 and not cfg.is_mla
            and cfg.causal and not cfg.post_norm and (cfg.is_moe or inter % 64 == 0)
            and cfg.hidden_act in L.ACT_IDS and cfg.hidden_size % 8 == 0)


def pack_attention(cfg: ModelConfig, src, i: int, rank: int, world: int, fused: bool, q_only: bool = False):
    """``q_only``: a shared-KV layer (ModelConfig.kv_donor): only the query projection is packed, n_kv is 0."""
    p = layer_prefix(i)
    D = cfg.head_dim
    if cfg.is_mla:   # projections live in models/mla.py; only o_proj (row-parallel over heads * v) is packed here
        wo = shard_tensor(p + "o_proj", src.get(p + "o_proj"), rank, world, head_dim=cfg.v_head_dim)
        empty = torch.zeros((0, cfg.hidden_size), dtype=wo.dtype)
        return empty, None, None, None, wo.contiguous(), src.get(p + "input_norm").float().contiguous(), \
            cfg.num_heads // world, 0
    sh = lambda n: shard_tensor(n, src.get(p + n), rank, world, head_dim=D)
    if cfg.num_kv_heads < world:
        # Fewer KV heads than ranks: a KV head is replicated over the world / num_kv_heads ranks whose query heads use
        # it. Rank r holds query heads [r * Hq/world, ...), all of which belong to KV head r * Hkv // world.
        if world % cfg.num_kv_heads:
            raise ValueError(f"kv heads {cfg.num_kv_heads} must divide tp={world} to be replicated")
        kvh = rank * cfg.num_kv_heads // world
        kv_sh = lambda n: src.get(p + n)[kvh * D:(kvh + 1) * D].contiguous()
    else:
        kv_sh = sh
    q = sh("q_proj")
    k, v = (q[:0], q[:0]) if q_only else (kv_sh("k_proj"), kv_sh("v_proj"))
    wqkv = torch.cat([q, k, v], 0)
    input_norm = src.get(p + "input_norm").float()
    if fused:
        wqkv = _fold(wqkv, input_norm, cfg.norm_one_plus_w)
    bias = None
    if cfg.attention_bias and src.has(p + "q_proj_bias"):
        parts = [sh("q_proj_bias")] + ([] if q_only else [kv_sh("k_proj_bias"), kv_sh("v_proj_bias")])
        bias = torch.cat(parts).float().contiguous()
    qn = src.get(p + "q_norm").float().contiguous() if cfg.qk_norm else None
    kn = src.get(p + "k_norm").float().contiguous() if cfg.qk_norm and not q_only else None
    wo = sh("o_proj")
    return wqkv.contiguous(), bias, qn, kn, wo.contiguous(), input_norm.contiguous(), q.shape[0] // D, k.shape[0] // D


def glu_tile_width(inter: int, sms: int = 148) -> int:
    """Tile width of the packed gate/up weight. 192 when that yields one nearly full wave of CTAs
    (e.g. 128 tiles for intermediate 12288), else the widest power-of-two tile that divides."""
    if inter % 96 == 0 and 0.8 * sms <= (2 * inter) // 192 <= sms:
        return 192
    if inter % 128 == 0 and (2 * inter) // 256 >= 32:
        return 256
    # a narrow gate/up weight (a tensor-parallel shard): 128-wide tiles give twice the tiles, and the decode-shaped
    # split-K paths (cluster reduce, parked partial tiles) exist for 128-wide tiles only
    return 128


def pack_mlp(cfg: ModelConfig, src, prefix: str, rank: int, world: int, fused: bool, norm_w=None, bn=None):
    g = shard_tensor(prefix + "gate_proj", src.get(prefix + "gate_proj"), rank, world)
    u = shard_tensor(prefix + "up_proj", src.get(prefix + "up_proj"), rank, world)
    d = shard_tensor(prefix + "down_proj", src.get(prefix + "down_proj"), rank, world)
    if getattr(cfg, "static_compression", "") == "dead_columns" and world == 1:
        # load-time static compression (loader/static_compression.py): neurons that cannot contribute leave all three
        # matrices; the kept count stays a multiple of 128 so that every tile width still divides it
        from ..loader.static_compression import prune_dead_ffn_columns
        g, u, d, _ = prune_dead_ffn_columns(g, u, d, multiple_of=128)
    inter = g.shape[0]
    if fused:
        # 256-wide tiles (128 gate + 128 up rows): a weight tile pulled into shared memory once serves
        # the most rows; split-K supplies the parallelism at decode batch sizes
        bn = bn or glu_tile_width(inter)
        if norm_w is not None:
            g, u = _fold(g, norm_w, cfg.norm_one_plus_w), _fold(u, norm_w, cfg.norm_one_plus_w)
        return L.interleave_gate_up(g, u, bn), d.contiguous(), bn
    return torch.cat([g, u], 0).contiguous(), d.contiguous(), 0


def pack_dense_layer(cfg: ModelConfig, src, i: int, rank: int = 0, world: int = 1, fused: Optional[bool] = None):
    fused = can_fuse(cfg, world) if fused is None else fused
    p = layer_prefix(i)
    donor = cfg.kv_donor(i) if not cfg.is_mla else None
    wqkv, bias, qn, kn, wo, input_norm, n_q, n_kv = pack_attention(cfg, src, i, rank, world, fused, q_only=donor is not None)
    post = src.get(p + "post_attn_norm").float().contiguous()
    lw = DenseLayerWeights(fused=fused, wqkv=wqkv, qkv_bias=bias, q_norm=qn, k_norm=kn, wo=wo, w_gate_up=None,
                           w_down=None, input_norm=input_norm, post_attn_norm=post, n_q=n_q, n_kv=n_kv)
    lw.kv_donor = donor
    if not cfg.layer_is_moe(i):
        lw.w_gate_up, lw.w_down, lw.glu_bn = pack_mlp(cfg, src, p, rank, world, fused, post if fused else None)
    return lw
