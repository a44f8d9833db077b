"""Model configuration: one dataclass filled from HF ``config.json``, GGUF metadata or tensor shapes.

Reference parity: ``ModelConfig`` / ``ModelGeometry`` with a field registry of HF and GGUF keys and the
RoPE-scaling family (src/model_config_fragments/types.inc.rs:19-118,285-322,404-529;
field_registry.inc.rs:70-1450); config.json is optional there too, so every field can also be
derived from tensor shapes (see ``models/arch.py``).
"""
from __future__ import annotations

import dataclasses
import json
import math
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Dict, List, Optional


@dataclass
class RopeScaling:
    """linear | dynamic | yarn | longrope | ntk | llama3 (types.inc.rs:285-322)."""
    kind: str = "none"
    factor: float = 1.0
    original_max_position: int = 0
    low_freq_factor: float = 1.0
    high_freq_factor: float = 4.0
    beta_fast: float = 32.0
    beta_slow: float = 1.0
    mscale: float = 1.0
    mscale_all_dim: float = 0.0
    long_factor: Optional[List[float]] = None
    short_factor: Optional[List[float]] = None
    attention_factor: Optional[float] = None


@dataclass
class ModelConfig:
    arch: str = "llama"
    kind: str = "chat"  # chat | embedding | reranker | classifier
    hidden_size: int = 0
    num_layers: int = 0
    num_heads: int = 0
    num_kv_heads: int = 0
    head_dim: int = 0
    intermediate_size: int = 0
    vocab_size: int = 0
    max_position_embeddings: int = 4096
    rms_norm_eps: float = 1e-5
    norm_type: str = "rms"  # rms | layer
    norm_one_plus_w: bool = False  # Gemma (1+w) variant
    rope_theta: float = 10000.0
    rope_local_theta: float = 0.0  # dual-RoPE models: theta of sliding layers
    partial_rotary_factor: float = 1.0
    rope_scaling: RopeScaling = field(default_factory=RopeScaling)
    tie_word_embeddings: bool = False
    qk_norm: bool = False  # per-head RMSNorm with weight (Qwen3)
    qk_norm_eps: float = 1e-6
    attention_bias: bool = False
    mlp_bias: bool = False
    hidden_act: str = "silu"
    sliding_window: int = 0
    num_kv_shared_layers: int = 0      # trailing layers that reuse an earlier layer's KV cache (see kv_donor)
    # Gemma-3n residual structure (models/gemma_ops.py): AltUp keeps ``altup_num_inputs`` residual streams and runs the
    # layer on one of them, LAuReL adds a low-rank path beside the attention, PLE feeds a per-layer token embedding
    altup_num_inputs: int = 0
    altup_active_idx: int = 0
    laurel_rank: int = 0
    ple_dim: int = 0
    static_compression: str = ""       # "dead_columns": drop dead FFN neurons when a layer is packed (loader option)
    attention_pattern: Optional[List[int]] = None  # per layer: 1 = sliding, 0 = global
    attention_sinks: bool = False
    embedding_scale: float = 1.0
    logit_softcap: float = 0.0
    attn_scale: float = 0.0  # 0 -> 1/sqrt(head_dim)
    post_norm: bool = False  # encoder-style post-LN residual blocks
    causal: bool = True
    # MoE
    num_experts: int = 0
    num_experts_per_tok: int = 0
    moe_intermediate_size: int = 0
    num_shared_experts: int = 0
    shared_expert_intermediate_size: int = 0
    norm_topk_prob: bool = True
    first_k_dense: int = 0
    moe_layer_freq: int = 1
    router_scoring: str = "softmax"  # softmax | sigmoid
    routed_scaling_factor: float = 1.0
    n_group: int = 0
    topk_group: int = 0
    # MLA
    q_lora_rank: int = 0
    kv_lora_rank: int = 0
    qk_nope_head_dim: int = 0
    qk_rope_head_dim: int = 0
    v_head_dim: int = 0
    # MTP
    num_mtp_layers: int = 0
    # encoder / heads
    type_vocab_size: int = 0
    position_embedding_type: str = "rope"  # rope | absolute | none
    layer_norm_eps: float = 1e-12
    num_labels: int = 0
    pooling: str = "mean"  # mean | cls | last
    pad_token_id: int = 0
    bos_token_id: int = 1
    eos_token_ids: List[int] = field(default_factory=list)
    # quantisation hints
    quant: str = ""  # "", fp8, mxfp8, nvfp4, mxfp4, awq, gptq, gguf
    kv_cache_dtype: str = "bf16"
    kv_cache_block_size: int = 16
    dtype: str = "bf16"
    extra: Dict[str, Any] = field(default_factory=dict)

    # ----------------------------------------------------------------------------------------
    def __post_init__(self):
        if self.num_kv_heads == 0:
            self.num_kv_heads = self.num_heads
        if self.head_dim == 0 and self.num_heads:
            self.head_dim = self.hidden_size // self.num_heads

    @property
    def is_moe(self) -> bool:
        return self.num_experts > 0

    @property
    def is_mla(self) -> bool:
        return self.kv_lora_rank > 0

    @property
    def is_encoder(self) -> bool:
        return not self.causal

    @property
    def rotary_dim(self) -> int:
        if self.position_embedding_type != "rope":
            return 0
        d = self.qk_rope_head_dim if self.is_mla else self.head_dim
        r = int(d * self.partial_rotary_factor)
        return r - (r % 2)

    @property
    def q_size(self) -> int:
        return self.num_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.num_kv_heads * self.head_dim

    def layer_is_moe(self, layer: int) -> bool:
        return self.is_moe and layer >= self.first_k_dense and (layer % max(self.moe_layer_freq, 1) == 0
                                                                 or self.moe_layer_freq <= 1)

    @property
    def gemma3n_structure(self) -> bool:
        return self.altup_num_inputs > 1 or self.laurel_rank > 0 or self.ple_dim > 0

    def kv_donor(self, layer: int):
        """Shared-KV layers (the last ``num_kv_shared_layers`` of the stack) project no keys or values of their own:
        they attend over the cache of the last earlier layer of the same attention kind (sliding-window or global).
        Returns that layer's index, or None for a layer that owns its cache (src/arch/resolve.rs:16-455 resolves the
        same donor map)."""
        first_shared = self.num_layers - int(self.num_kv_shared_layers or 0)
        if self.num_kv_shared_layers <= 0 or layer < first_shared:
            return None
        kind = self.layer_window(layer) > 0
        for d in range(first_shared - 1, -1, -1):
            if (self.layer_window(d) > 0) == kind:
                return d
        return first_shared - 1

    def layer_window(self, layer: int) -> int:
        if not self.sliding_window:
            return 0
        if self.attention_pattern is None:
            return self.sliding_window
        return self.sliding_window if self.attention_pattern[layer % len(self.attention_pattern)] else 0

    def attention_scale(self) -> float:
        if self.attn_scale:
            return self.attn_scale
        d = (self.qk_nope_head_dim + self.qk_rope_head_dim) if self.is_mla else self.head_dim
        s = 1.0 / math.sqrt(d)
        rs = self.rope_scaling
        if self.is_mla and rs.kind == "yarn" and rs.mscale_all_dim:
            m = 0.1 * rs.mscale_all_dim * math.log(rs.factor) + 1.0 if rs.factor > 1 else 1.0
            s = s * m * m
        return s

    def param_count(self) -> int:
        h, L = self.hidden_size, self.num_layers
        attn = h * (self.q_size + 2 * self.kv_size) + self.q_size * h
        if self.is_mla:
            qd = self.qk_nope_head_dim + self.qk_rope_head_dim
            q = (h * self.q_lora_rank + self.q_lora_rank * self.num_heads * qd) if self.q_lora_rank else h * self.num_heads * qd
            attn = q + h * (self.kv_lora_rank + self.qk_rope_head_dim) + self.kv_lora_rank * self.num_heads * (
                self.qk_nope_head_dim + self.v_head_dim) + self.num_heads * self.v_head_dim * h
        dense = 3 * h * self.intermediate_size
        total = 0
        for l in range(L):
            total += attn
            if self.layer_is_moe(l):
                total += self.num_experts * 3 * h * self.moe_intermediate_size + h * self.num_experts
                total += self.num_shared_experts * 3 * h * (self.shared_expert_intermediate_size or self.moe_intermediate_size)
            else:
                total += dense
        total += self.vocab_size * h * (1 if self.tie_word_embeddings else 2)
        return total

    def kv_bytes_per_token(self, tp: int = 1) -> int:
        esz = 1 if self.kv_cache_dtype in ("fp8", "fp8_e4m3") else 2
        if self.is_mla:
            return self.num_layers * (self.kv_lora_rank + self.qk_rope_head_dim) * esz
        return self.num_layers * 2 * max(1, self.num_kv_heads // tp) * self.head_dim * esz

    def to_dict(self) -> Dict[str, Any]:
        return dataclasses.asdict(self)

    # ----------------------------------------------------------------------------------------
    @staticmethod
    def from_hf_dict(d: Dict[str, Any]) -> "ModelConfig":
        """HF ``config.json`` -> ModelConfig (keys per the reference's field registry)."""
        tc = d.get("text_config") or d
        arch = (d.get("model_type") or tc.get("model_type") or "llama").lower()
        g = lambda *keys, default=None: next((tc[k] for k in keys if k in tc and tc[k] is not None), default)
        hidden = g("hidden_size", "n_embd", "d_model", default=0)
        heads = g("num_attention_heads", "n_head", default=0)
        cfg = ModelConfig(
            arch=arch, hidden_size=hidden, num_layers=g("num_hidden_layers", "n_layer", default=0),
            num_heads=heads, num_kv_heads=g("num_key_value_heads", default=heads),
            head_dim=g("head_dim", default=(hidden // heads if heads else 0)),
            intermediate_size=g("intermediate_size", "n_inner", default=0) or 4 * hidden,
            vocab_size=g("vocab_size", default=0),
            max_position_embeddings=g("max_position_embeddings", "n_positions", default=4096),
            rms_norm_eps=g("rms_norm_eps", "layer_norm_epsilon", "layer_norm_eps", default=1e-12),
            rope_theta=float(g("rope_theta", default=10000.0)),
            rope_local_theta=float(g("rope_local_base_freq", default=0.0) or 0.0),
            partial_rotary_factor=float(g("partial_rotary_factor", default=1.0)),
            tie_word_embeddings=bool(d.get("tie_word_embeddings", tc.get("tie_word_embeddings", False))),
            attention_bias=bool(g("attention_bias", "qkv_bias", default=arch in ("qwen2",))),
            mlp_bias=bool(g("mlp_bias", default=False)),
            hidden_act=str(g("hidden_act", "hidden_activation", "activation_function", default="silu")),
            sliding_window=int(g("sliding_window", default=0) or 0) if g("use_sliding_window", default=True) else 0,
            num_kv_shared_layers=int(g("num_kv_shared_layers", default=0) or 0),
            altup_num_inputs=int(g("altup_num_inputs", default=0) or 0),
            altup_active_idx=int(g("altup_active_idx", default=0) or 0),
            laurel_rank=int(g("laurel_rank", default=0) or 0),
            ple_dim=int(g("hidden_size_per_layer_input", default=0) or 0),
            num_experts=int(g("num_experts", "num_local_experts", "n_routed_experts", default=0) or 0),
            num_experts_per_tok=int(g("num_experts_per_tok", default=0) or 0),
            moe_intermediate_size=int(g("moe_intermediate_size", default=0) or 0),
            num_shared_experts=int(g("n_shared_experts", default=0) or 0),
            norm_topk_prob=bool(g("norm_topk_prob", default=True)),
            first_k_dense=int(g("first_k_dense_replace", default=0) or 0),
            q_lora_rank=int(g("q_lora_rank", default=0) or 0),
            kv_lora_rank=int(g("kv_lora_rank", default=0) or 0),
            qk_nope_head_dim=int(g("qk_nope_head_dim", default=0) or 0),
            qk_rope_head_dim=int(g("qk_rope_head_dim", default=0) or 0),
            v_head_dim=int(g("v_head_dim", default=0) or 0),
            num_mtp_layers=int(g("num_nextn_predict_layers", default=0) or 0),
            type_vocab_size=int(g("type_vocab_size", default=0) or 0),
            num_labels=int(d.get("num_labels", len(d.get("id2label", {}) or {})) or 0),
            pad_token_id=int(g("pad_token_id", default=0) or 0),
            bos_token_id=int(g("bos_token_id", default=1) or 0),
            logit_softcap=float(g("final_logit_softcapping", default=0.0) or 0.0),
            routed_scaling_factor=float(g("routed_scaling_factor", default=1.0) or 1.0),
            n_group=int(g("n_group", default=0) or 0), topk_group=int(g("topk_group", default=0) or 0),
        )
        eos = g("eos_token_id", default=None)
        cfg.eos_token_ids = [] if eos is None else ([int(e) for e in eos] if isinstance(eos, list) else [int(eos)])
        if arch in ("qwen3", "qwen3_moe"):
            cfg.qk_norm = True
        if arch in ("deepseek_v3", "deepseek_v2"):
            cfg.router_scoring = str(g("scoring_func", default="sigmoid" if arch == "deepseek_v3" else "softmax"))
            cfg.head_dim = cfg.qk_nope_head_dim + cfg.qk_rope_head_dim
        if arch in ("gemma", "gemma2", "gemma3", "gemma3_text"):
            cfg.norm_one_plus_w = True
            cfg.embedding_scale = math.sqrt(hidden)
        if arch in ("gpt_oss",):
            cfg.attention_sinks = True
        if arch in ("bert", "xlm-roberta", "roberta", "modernbert", "new", "nomic_bert"):
            cfg.causal = False
            cfg.kind = "embedding"
            cfg.norm_type = "layer"
            cfg.post_norm = arch != "modernbert"
            cfg.position_embedding_type = str(g("position_embedding_type", default="absolute"))
            cfg.layer_norm_eps = float(g("layer_norm_eps", default=1e-12))
            cfg.hidden_act = str(g("hidden_act", default="gelu"))
            cfg.pooling = "cls" if cfg.num_labels else "mean"
        lt = g("layer_types", default=None)
        if lt:
            cfg.attention_pattern = [1 if "sliding" in str(t) else 0 for t in lt]
        rs = g("rope_scaling", default=None)
        if isinstance(rs, dict):
            kind = str(rs.get("rope_type", rs.get("type", "none"))).lower()
            cfg.rope_scaling = RopeScaling(
                kind={"default": "none", "su": "longrope"}.get(kind, kind), factor=float(rs.get("factor", 1.0)),
                original_max_position=int(rs.get("original_max_position_embeddings", 0) or 0),
                low_freq_factor=float(rs.get("low_freq_factor", 1.0)),
                high_freq_factor=float(rs.get("high_freq_factor", 4.0)),
                beta_fast=float(rs.get("beta_fast", 32.0)), beta_slow=float(rs.get("beta_slow", 1.0)),
                mscale=float(rs.get("mscale", 1.0)), mscale_all_dim=float(rs.get("mscale_all_dim", 0.0)),
                long_factor=rs.get("long_factor"), short_factor=rs.get("short_factor"),
                attention_factor=rs.get("attention_factor"))
        qc = d.get("quantization_config")
        if isinstance(qc, dict):
            cfg.quant = str(qc.get("quant_method", "")).lower()
            cfg.extra["quantization_config"] = qc
        return cfg

    @staticmethod
    def from_json_file(path) -> "ModelConfig":
        return ModelConfig.from_hf_dict(json.loads(Path(path).read_text()))

    @staticmethod
    def from_gguf_metadata(md: Dict[str, Any]) -> "ModelConfig":
        """GGUF key/value metadata -> ModelConfig (``<arch>.*`` keys; src/loader/gguf/reader.rs:190-570)."""
        arch = str(md.get("general.architecture", "llama"))
        k = lambda name, default=None: md.get(f"{arch}.{name}", default)
        hidden = int(k("embedding_length", 0))
        heads = int(k("attention.head_count", 0))
        kvh = k("attention.head_count_kv", heads)
        if isinstance(kvh, (list, tuple)):
            kvh = max(kvh)
        vocab = md.get(f"{arch}.vocab_size")
        if vocab is None:
            toks = md.get("tokenizer.ggml.tokens")
            vocab = len(toks) if toks is not None else 0
        cfg = ModelConfig(
            arch={"qwen3moe": "qwen3_moe", "deepseek2": "deepseek_v3"}.get(arch, arch), hidden_size=hidden,
            num_layers=int(k("block_count", 0)), num_heads=heads, num_kv_heads=int(kvh),
            head_dim=int(k("attention.key_length", hidden // heads if heads else 0)),
            intermediate_size=int(k("feed_forward_length", 0) if not isinstance(k("feed_forward_length", 0), (list, tuple))
                                  else max(k("feed_forward_length"))),
            vocab_size=int(vocab), max_position_embeddings=int(k("context_length", 4096)),
            rms_norm_eps=float(k("attention.layer_norm_rms_epsilon", k("attention.layer_norm_epsilon", 1e-5))),
            rope_theta=float(k("rope.freq_base", 10000.0)),
            num_experts=int(k("expert_count", 0) or 0), num_experts_per_tok=int(k("expert_used_count", 0) or 0),
            moe_intermediate_size=int(k("expert_feed_forward_length", 0) or 0),
            num_shared_experts=int(k("expert_shared_count", 0) or 0),
            first_k_dense=int(k("leading_dense_block_count", 0) or 0),
            q_lora_rank=int(k("attention.q_lora_rank", 0) or 0), kv_lora_rank=int(k("attention.kv_lora_rank", 0) or 0),
            num_mtp_layers=int(k("nextn_predict_layers", 0) or 0),
            sliding_window=int(k("attention.sliding_window", 0) or 0),
            bos_token_id=int(md.get("tokenizer.ggml.bos_token_id", 1)),
            pad_token_id=int(md.get("tokenizer.ggml.padding_token_id", 0)),
        )
        rd = k("rope.dimension_count")
        if rd and cfg.head_dim:
            cfg.partial_rotary_factor = float(rd) / cfg.head_dim
        if "tokenizer.ggml.eos_token_id" in md:
            cfg.eos_token_ids = [int(md["tokenizer.ggml.eos_token_id"])]
        st = k("rope.scaling.type")
        if st and st != "none":
            cfg.rope_scaling = RopeScaling(kind=str(st), factor=float(k("rope.scaling.factor", 1.0)),
                                           original_max_position=int(k("rope.scaling.original_context_length", 0) or 0))
        if cfg.arch in ("qwen3", "qwen3_moe"):
            cfg.qk_norm = True
        cfg.quant = "gguf"
        return cfg


# ------------------------------------------------------------------------------------------------
# Named shapes used by the benchmarks and tests (random-init weights of these architectures)
# ------------------------------------------------------------------------------------------------
def preset(name: str) -> ModelConfig:
    n = name.lower()
    if n in ("smollm2-135m", "smollm2"):
        return ModelConfig(arch="llama", hidden_size=576, num_layers=30, num_heads=9, num_kv_heads=3, head_dim=64,
                           intermediate_size=1536, vocab_size=49152, rope_theta=1e5, rms_norm_eps=1e-5,
                           tie_word_embeddings=True, max_position_embeddings=8192, eos_token_ids=[2])
    if n in ("qwen3-8b",):
        return ModelConfig(arch="qwen3", hidden_size=4096, num_layers=36, num_heads=32, num_kv_heads=8, head_dim=128,
                           intermediate_size=12288, vocab_size=151936, rope_theta=1e6, rms_norm_eps=1e-6, qk_norm=True,
                           max_position_embeddings=40960, eos_token_ids=[151645])
    if n in ("qwen3-30b-a3b",):
        return ModelConfig(arch="qwen3_moe", hidden_size=2048, num_layers=48, num_heads=32, num_kv_heads=4,
                           head_dim=128, intermediate_size=6144, vocab_size=151936, rope_theta=1e6, rms_norm_eps=1e-6,
                           qk_norm=True, num_experts=128, num_experts_per_tok=8, moe_intermediate_size=768,
                           norm_topk_prob=True, max_position_embeddings=40960, quant="mxfp8",
                           eos_token_ids=[151645])
    if n in ("llama-3-70b", "llama3-70b"):
        return ModelConfig(arch="llama", hidden_size=8192, num_layers=80, num_heads=64, num_kv_heads=8, head_dim=128,
                           intermediate_size=28672, vocab_size=128256, rope_theta=5e5, rms_norm_eps=1e-5,
                           max_position_embeddings=8192 + 1024, quant="nvfp4", kv_cache_dtype="fp8",
                           eos_token_ids=[128001])
    if n in ("deepseek-v3",):
        return ModelConfig(arch="deepseek_v3", hidden_size=7168, num_layers=61, num_heads=128, num_kv_heads=128,
                           head_dim=192, intermediate_size=18432, vocab_size=129280, rope_theta=1e4, rms_norm_eps=1e-6,
                           num_experts=256, num_experts_per_tok=8, moe_intermediate_size=2048, num_shared_experts=1,
                           first_k_dense=3, q_lora_rank=1536, kv_lora_rank=512, qk_nope_head_dim=128,
                           qk_rope_head_dim=64, v_head_dim=128, router_scoring="sigmoid", routed_scaling_factor=2.5,
                           n_group=8, topk_group=4, max_position_embeddings=4096, quant="fp8", eos_token_ids=[1])
    if n in ("tiny-llama", "tiny"):
        return ModelConfig(arch="llama", hidden_size=256, num_layers=2, num_heads=2, num_kv_heads=1, head_dim=128,
                           intermediate_size=512, vocab_size=1024, rope_theta=1e4, max_position_embeddings=2048,
                           eos_token_ids=[2])
    if n in ("tiny-qwen3",):
        return ModelConfig(arch="qwen3", hidden_size=256, num_layers=2, num_heads=4, num_kv_heads=2, head_dim=128,
                           intermediate_size=512, vocab_size=1024, rope_theta=1e6, rms_norm_eps=1e-6, qk_norm=True,
                           max_position_embeddings=2048, eos_token_ids=[2])
    if n in ("tiny-moe",):
        return ModelConfig(arch="qwen3_moe", hidden_size=256, num_layers=2, num_heads=4, num_kv_heads=2, head_dim=128,
                           intermediate_size=512, vocab_size=1024, rope_theta=1e6, rms_norm_eps=1e-6, qk_norm=True,
                           num_experts=8, num_experts_per_tok=2, moe_intermediate_size=128,
                           max_position_embeddings=2048, eos_token_ids=[2])
    if n in ("tiny-mla",):
        return ModelConfig(arch="deepseek_v3", hidden_size=256, num_layers=2, num_heads=4, num_kv_heads=4,
                           head_dim=48, intermediate_size=512, vocab_size=1024, rms_norm_eps=1e-6, q_lora_rank=64,
                           kv_lora_rank=32, qk_nope_head_dim=32, qk_rope_head_dim=16, v_head_dim=32, num_experts=8,
                           num_experts_per_tok=2, moe_intermediate_size=128, num_shared_experts=1, first_k_dense=1,
                           router_scoring="sigmoid", max_position_embeddings=2048, eos_token_ids=[2])
    if n in ("tiny-bert",):
        return ModelConfig(arch="bert", kind="embedding", hidden_size=128, num_layers=2, num_heads=2, num_kv_heads=2,
                           head_dim=64, intermediate_size=256, vocab_size=512, causal=False, norm_type="layer",
                           post_norm=True, position_embedding_type="absolute", hidden_act="gelu", type_vocab_size=2,
                           max_position_embeddings=512, attention_bias=True, mlp_bias=True)
    raise KeyError(f"unknown preset {name}")
