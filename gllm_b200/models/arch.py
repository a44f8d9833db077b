"""Tensor-driven architecture analysis: derive model features (and, when ``config.json`` is absent, the whole
``ModelConfig``) from which tensor roles exist and their shapes.

Reference parity: ``analyze_architecture`` (src/arch/auto_graph_fragments/types.inc.rs:45-397): decoder vs
encoder from OutputHead / tied embedding, layer count, RoPE, per-head q/k norm, biases, attention sinks, norm
type, FFN type (SwiGLU / GeGLU / standard / MoE), shared experts, expert count from the router shape, MLA
dimensions, classifier head; arch alias table (src/arch/registry.rs:12-70).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Optional, Tuple

from ..loader.name_map import TensorRole, match_tensor_role
from .config import ModelConfig

ARCH_ALIASES = {
    "llama": "llama", "llama3": "llama", "mistral": "llama", "mistral3": "llama", "smollm": "llama", "smollm2": "llama",
    "qwen2": "qwen2", "qwen3": "qwen3", "qwen3_moe": "qwen3_moe", "qwen3moe": "qwen3_moe", "phi3": "phi3", "phi4": "phi3",
    "glm4": "glm4", "gemma": "gemma", "gemma2": "gemma", "gemma3": "gemma", "gemma4": "gemma",
    "deepseek_v2": "deepseek_v3", "deepseek_v3": "deepseek_v3", "deepseek2": "deepseek_v3", "deepseek": "deepseek_v3",
    "gpt_oss": "gpt_oss", "gptoss": "gpt_oss", "gpt-oss": "gpt_oss", "mixtral": "mixtral",
    "bert": "bert", "xlm-roberta": "bert", "xlmr": "bert", "roberta": "bert", "bge": "bert", "e5": "bert",
    "modernbert": "modernbert", "siglip": "siglip", "usm": "usm", "gpt2": "gpt2",
}


def canonical_arch(name: str) -> str:
    return ARCH_ALIASES.get(name.lower().replace("forcausallm", "").replace("model", ""), name.lower())


@dataclass
class ArchFeatures:
    is_decoder: bool = True
    num_layers: int = 0
    hidden_size: int = 0
    vocab_size: int = 0
    tied_embeddings: bool = False
    has_rope: bool = True
    qk_norm: bool = False
    attention_bias: bool = False
    mlp_bias: bool = False
    attention_sinks: bool = False
    fused_qkv: bool = False
    fused_gate_up: bool = False
    norm_type: str = "rms"
    ffn_type: str = "swiglu"  # swiglu | standard | moe
    num_experts: int = 0
    shared_experts: bool = False
    moe_intermediate: int = 0
    intermediate: int = 0
    q_out: int = 0
    kv_out: int = 0
    is_mla: bool = False
    q_lora_rank: int = 0
    kv_lora_rank: int = 0
    mla_rope_dim: int = 0
    has_classifier: bool = False
    num_labels: int = 0
    has_position_embeddings: bool = False
    max_positions: int = 0
    type_vocab: int = 0
    first_moe_layer: int = -1
    roles: Dict[str, int] = field(default_factory=dict)


def analyze_architecture(shapes: Dict[str, Tuple[int, ...]]) -> ArchFeatures:
    """shapes: external tensor name -> shape."""
    f = ArchFeatures()
    layers = set()
    experts = set()
    has_head = False
    for name, shape in shapes.items():
        role, layer, canon, suffix = match_tensor_role(name)
        f.roles[role.value] = f.roles.get(role.value, 0) + 1
        if layer is not None:
            layers.add(layer)
        is_w = suffix in ("", ".weight", ".qweight", "_blocks")
        if role == TensorRole.EMBEDDING and is_w:
            f.vocab_size, f.hidden_size = int(shape[0]), int(shape[1])
        elif role == TensorRole.OUTPUT_HEAD:
            has_head = True
        elif role == TensorRole.POSITION_EMBEDDING:
            f.has_position_embeddings, f.max_positions = True, int(shape[0])
        elif role == TensorRole.TOKEN_TYPE_EMBEDDING:
            f.type_vocab = int(shape[0])
        elif role in (TensorRole.ATTN_Q_NORM, TensorRole.ATTN_K_NORM):
            f.qk_norm = True
        elif role == TensorRole.ATTN_SINKS:
            f.attention_sinks = True
        elif role == TensorRole.ATTN_FUSED_QKV:
            f.fused_qkv = True
        elif role == TensorRole.ATTN_QUERY:
            if suffix in (".bias", "_bias"):
                f.attention_bias = True
            elif is_w:
                f.q_out = int(shape[0])
        elif role == TensorRole.ATTN_KEY and is_w:
            f.kv_out = int(shape[0])
        elif role in (TensorRole.FFN_GATE, TensorRole.FFN_UP) and is_w:
            f.intermediate = int(shape[0])
            if suffix in (".bias", "_bias"):
                f.mlp_bias = True
        elif role == TensorRole.FFN_FUSED_GATE_UP:
            f.fused_gate_up = True
            f.intermediate = int(shape[0]) // 2
        elif role == TensorRole.MOE_ROUTER and is_w:
            f.num_experts = max(f.num_experts, int(shape[0]))
            if layer is not None:
                f.first_moe_layer = layer if f.first_moe_layer < 0 else min(f.first_moe_layer, layer)
        elif role == TensorRole.MOE_EXPERT_GATE and is_w:
            f.moe_intermediate = int(shape[-2]) if len(shape) == 3 else int(shape[0])
            if canon and ".experts." in canon and "stacked" not in canon:
                experts.add(int(canon.split(".experts.")[1].split(".")[0]))
        elif role in (TensorRole.MOE_SHARED_GATE,):
            f.shared_experts = True
        elif role == TensorRole.MLA_KV_COMPRESS and is_w:
            f.is_mla = True
        elif role == TensorRole.MLA_KV_NORM:
            f.kv_lora_rank = int(shape[0])
        elif role == TensorRole.MLA_Q_NORM:
            f.q_lora_rank = int(shape[0])
        elif role == TensorRole.CLASSIFIER and is_w:
            f.has_classifier, f.num_labels = True, int(shape[0])
        elif role in (TensorRole.INPUT_NORM, TensorRole.POST_ATTN_NORM) and suffix in (".bias", "_bias"):
            f.norm_type = "layer"
    f.num_layers = (max(layers) + 1) if layers else 0
    if experts:
        f.num_experts = max(f.num_experts, max(experts) + 1)
    # decoder if it has an output head, or its (large) embedding doubles as one (tied)
    f.tied_embeddings = not has_head and f.vocab_size > 10000 and not f.has_position_embeddings
    f.is_decoder = has_head or f.tied_embeddings
    if f.has_position_embeddings:
        f.has_rope = False
        f.norm_type = "layer"
    if f.num_experts:
        f.ffn_type = "moe"
    elif f.roles.get(TensorRole.FFN_GATE.value, 0) == 0 and not f.fused_gate_up:
        f.ffn_type = "standard"
    if f.is_mla:
        for name, shape in shapes.items():
            role, _, _, suffix = match_tensor_role(name)
            if role == TensorRole.MLA_KV_COMPRESS and suffix in ("", ".weight"):
                f.mla_rope_dim = int(shape[0]) - f.kv_lora_rank
                break
    return f


def config_from_features(f: ArchFeatures, arch: str = "", head_dim: int = 0) -> ModelConfig:
    """Best-effort ModelConfig when no config.json / GGUF metadata is available."""
    hd = head_dim or (128 if f.q_out % 128 == 0 and f.hidden_size >= 2048 else 64)
    heads = max(1, f.q_out // hd) if f.q_out else max(1, f.hidden_size // hd)
    kvh = max(1, f.kv_out // hd) if f.kv_out else heads
    arch = arch or ("qwen3_moe" if f.num_experts and f.qk_norm else "qwen3" if f.qk_norm else
                    "deepseek_v3" if f.is_mla else "bert" if not f.is_decoder else "llama")
    cfg = ModelConfig(arch=arch, hidden_size=f.hidden_size, num_layers=f.num_layers, num_heads=heads,
                      num_kv_heads=kvh, head_dim=hd, intermediate_size=f.intermediate or 4 * f.hidden_size,
                      vocab_size=f.vocab_size, tie_word_embeddings=f.tied_embeddings, qk_norm=f.qk_norm,
                      attention_bias=f.attention_bias, mlp_bias=f.mlp_bias, attention_sinks=f.attention_sinks,
                      num_experts=f.num_experts, moe_intermediate_size=f.moe_intermediate,
                      num_shared_experts=1 if f.shared_experts else 0, first_k_dense=max(f.first_moe_layer, 0),
                      q_lora_rank=f.q_lora_rank, kv_lora_rank=f.kv_lora_rank, qk_rope_head_dim=f.mla_rope_dim,
                      num_labels=f.num_labels, type_vocab_size=f.type_vocab)
    if not f.is_decoder:
        cfg.causal, cfg.kind, cfg.norm_type, cfg.post_norm = False, "embedding", "layer", True
        cfg.position_embedding_type = "absolute" if f.has_position_embeddings else "rope"
        cfg.hidden_act = "gelu"
        if f.max_positions:
            cfg.max_position_embeddings = f.max_positions
        if f.has_classifier:
            cfg.kind, cfg.pooling = "reranker" if f.num_labels == 1 else "classifier", "cls"
    if f.num_experts and not cfg.num_experts_per_tok:
        cfg.num_experts_per_tok = 8 if f.num_experts >= 64 else 2
    return cfg
