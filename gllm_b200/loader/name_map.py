"""External tensor names (HF, GGUF, BERT-family) -> canonical names and roles.

Reference parity: suffix-table role matcher (src/loader/fragments/types.inc.rs:260-608, enum
src/manifest/types.rs:11-140) and the external <-> canonical map (src/loader/name_map.rs:7-293,
src/weight_names.rs:19-540). Canonical names: ``embed_tokens``, ``final_norm``, ``lm_head``,
``L{n}.q_proj``, ``L{n}.experts.{e}.gate_proj`` ...
"""
from __future__ import annotations

import re
from enum import Enum
from typing import Dict, Optional, Tuple


class TensorRole(str, Enum):
    EMBEDDING = "embedding"
    POSITION_EMBEDDING = "position_embedding"
    TOKEN_TYPE_EMBEDDING = "token_type_embedding"
    EMBEDDING_NORM = "embedding_norm"
    OUTPUT_HEAD = "output_head"
    FINAL_NORM = "final_norm"
    ATTN_QUERY = "attn_query"
    ATTN_KEY = "attn_key"
    ATTN_VALUE = "attn_value"
    ATTN_OUTPUT = "attn_output"
    ATTN_FUSED_QKV = "attn_fused_qkv"
    ATTN_Q_NORM = "attn_q_norm"
    ATTN_K_NORM = "attn_k_norm"
    ATTN_SINKS = "attn_sinks"
    MLA_Q_COMPRESS = "mla_q_compress"
    MLA_Q_NORM = "mla_q_norm"
    MLA_Q_EXPAND = "mla_q_expand"
    MLA_KV_COMPRESS = "mla_kv_compress"
    MLA_KV_NORM = "mla_kv_norm"
    MLA_KV_EXPAND = "mla_kv_expand"
    INPUT_NORM = "input_norm"
    POST_ATTN_NORM = "post_attn_norm"
    PRE_FFN_NORM = "pre_ffn_norm"
    POST_FFN_NORM = "post_ffn_norm"
    FFN_GATE = "ffn_gate"
    FFN_UP = "ffn_up"
    FFN_DOWN = "ffn_down"
    FFN_FUSED_GATE_UP = "ffn_fused_gate_up"
    MOE_ROUTER = "moe_router"
    MOE_ROUTER_BIAS = "moe_router_bias"
    MOE_EXPERT_GATE = "moe_expert_gate"
    MOE_EXPERT_UP = "moe_expert_up"
    MOE_EXPERT_DOWN = "moe_expert_down"
    MOE_SHARED_GATE = "moe_shared_gate"
    MOE_SHARED_UP = "moe_shared_up"
    MOE_SHARED_DOWN = "moe_shared_down"
    CLASSIFIER = "classifier"
    POOLER = "pooler"
    UNKNOWN = "unknown"


# (regex on the part after the layer prefix, canonical suffix, role)
_LAYER_RULES = [
    (r"(self_attn|attention\.self|attention|attn)\.(q_proj|query|wq|q)$|^attn_q$", "q_proj", TensorRole.ATTN_QUERY),
    (r"(self_attn|attention\.self|attention|attn)\.(k_proj|key|wk|k)$|^attn_k$", "k_proj", TensorRole.ATTN_KEY),
    (r"(self_attn|attention\.self|attention|attn)\.(v_proj|value|wv|v)$|^attn_v$", "v_proj", TensorRole.ATTN_VALUE),
    (r"(self_attn|attention|attn)\.(o_proj|out_proj|wo|dense|output\.dense)$|^attn_output$", "o_proj",
     TensorRole.ATTN_OUTPUT),
    (r"(self_attn|attention|attn)\.(qkv_proj|query_key_value|c_attn|Wqkv)$|^attn_qkv$", "qkv_proj",
     TensorRole.ATTN_FUSED_QKV),
    (r"(self_attn|attn)\.q_norm$|^attn_q_norm$", "q_norm", TensorRole.ATTN_Q_NORM),
    (r"(self_attn|attn)\.k_norm$|^attn_k_norm$", "k_norm", TensorRole.ATTN_K_NORM),
    (r"(self_attn|attn)\.sinks$|^attn_sinks$", "sinks", TensorRole.ATTN_SINKS),
    (r"self_attn\.q_a_proj$|^attn_q_a$", "q_a_proj", TensorRole.MLA_Q_COMPRESS),
    (r"self_attn\.q_a_layernorm$|^attn_q_a_norm$", "q_a_norm", TensorRole.MLA_Q_NORM),
    (r"self_attn\.q_b_proj$|^attn_q_b$", "q_b_proj", TensorRole.MLA_Q_EXPAND),
    (r"self_attn\.kv_a_proj_with_mqa$|^attn_kv_a_mqa$", "kv_a_proj", TensorRole.MLA_KV_COMPRESS),
    (r"self_attn\.kv_a_layernorm$|^attn_kv_a_norm$", "kv_a_norm", TensorRole.MLA_KV_NORM),
    (r"self_attn\.kv_b_proj$|^attn_kv_b$", "kv_b_proj", TensorRole.MLA_KV_EXPAND),
    (r"^input_layernorm$|^attn_norm$|^ln_1$|^attention_norm$", "input_norm", TensorRole.INPUT_NORM),
    (r"^post_attention_layernorm$|^ffn_norm$|^ln_2$|^attention\.output\.LayerNorm$", "post_attn_norm",
     TensorRole.POST_ATTN_NORM),
    (r"^pre_feedforward_layernorm$", "pre_ffn_norm", TensorRole.PRE_FFN_NORM),
    (r"^post_feedforward_layernorm$|^output\.LayerNorm$", "post_ffn_norm", TensorRole.POST_FFN_NORM),
    (r"(mlp|feed_forward)\.(gate_proj|w1)$|^ffn_gate$", "gate_proj", TensorRole.FFN_GATE),
    (r"(mlp|feed_forward)\.(up_proj|w3|c_fc)$|^ffn_up$|^intermediate\.dense$", "up_proj", TensorRole.FFN_UP),
    (r"(mlp|feed_forward)\.(down_proj|w2|c_proj)$|^ffn_down$|^output\.dense$", "down_proj", TensorRole.FFN_DOWN),
    (r"mlp\.gate_up_proj$", "gate_up_proj", TensorRole.FFN_FUSED_GATE_UP),
    (r"(mlp|block_sparse_moe)\.(gate|router)$|^ffn_gate_inp$", "router", TensorRole.MOE_ROUTER),
    (r"mlp\.gate\.e_score_correction_bias$|^exp_probs_b$", "router_bias", TensorRole.MOE_ROUTER_BIAS),
    (r"(mlp|block_sparse_moe)\.experts\.(\d+)\.(gate_proj|w1)$", "experts.{e}.gate_proj", TensorRole.MOE_EXPERT_GATE),
    (r"(mlp|block_sparse_moe)\.experts\.(\d+)\.(up_proj|w3)$", "experts.{e}.up_proj", TensorRole.MOE_EXPERT_UP),
    (r"(mlp|block_sparse_moe)\.experts\.(\d+)\.(down_proj|w2)$", "experts.{e}.down_proj", TensorRole.MOE_EXPERT_DOWN),
    (r"^ffn_gate_exps$", "experts.stacked.gate_proj", TensorRole.MOE_EXPERT_GATE),
    (r"^ffn_up_exps$", "experts.stacked.up_proj", TensorRole.MOE_EXPERT_UP),
    (r"^ffn_down_exps$", "experts.stacked.down_proj", TensorRole.MOE_EXPERT_DOWN),
    (r"mlp\.shared_experts?\.gate_proj$|^ffn_gate_shexp$", "shared_expert.gate_proj", TensorRole.MOE_SHARED_GATE),
    (r"mlp\.shared_experts?\.up_proj$|^ffn_up_shexp$", "shared_expert.up_proj", TensorRole.MOE_SHARED_UP),
    (r"mlp\.shared_experts?\.down_proj$|^ffn_down_shexp$", "shared_expert.down_proj", TensorRole.MOE_SHARED_DOWN),
]
_LAYER_RULES = [(re.compile(p), c, r) for p, c, r in _LAYER_RULES]

_GLOBAL_RULES = [
    (r"(^|\.)(embed_tokens|wte|word_embeddings|tok_embeddings)$|^token_embd$", "embed_tokens", TensorRole.EMBEDDING),
    (r"(^|\.)(wpe|position_embeddings)$|^position_embd$", "position_embeddings", TensorRole.POSITION_EMBEDDING),
    (r"(^|\.)token_type_embeddings$|^token_types$", "token_type_embeddings", TensorRole.TOKEN_TYPE_EMBEDDING),
    (r"embeddings\.LayerNorm$|^token_embd_norm$", "embed_norm", TensorRole.EMBEDDING_NORM),
    (r"(^|\.)lm_head$|^output$", "lm_head", TensorRole.OUTPUT_HEAD),
    (r"(^|model\.|transformer\.)(norm|ln_f|final_layernorm)$|^output_norm$", "final_norm", TensorRole.FINAL_NORM),
    (r"^classifier(\.out_proj)?$|^score$", "classifier", TensorRole.CLASSIFIER),
    (r"^classifier\.dense$|(^|\.)pooler\.dense$", "pooler", TensorRole.POOLER),
]
_GLOBAL_RULES = [(re.compile(p), c, r) for p, c, r in _GLOBAL_RULES]

_LAYER_PREFIX = re.compile(r"^(?:model\.|language_model\.|text_model\.|transformer\.|bert\.|roberta\.|encoder\.)*(?:layers|h|layer|blocks|blk|encoder\.layer)\.(\d+)\.(.+)$")
# tensors of a multimodal checkpoint's towers and projectors are not the language model's: they have their own loaders
_NOT_LANGUAGE = re.compile(r"(^|\.)(vision_tower|vision_model|visual|audio_tower|audio_model|multi_modal_projector|"
                           r"embed_vision|embed_audio|mm_projector)\.")
_SUFFIXES = (".weight", ".bias", ".qweight", ".qzeros", ".scales", ".g_idx", ".weight_scale", ".weight_scale_2",
             ".weight_scale_inv", ".input_scale", "_blocks", "_scales", "_bias")


def split_suffix(name: str) -> Tuple[str, str]:
    for s in _SUFFIXES:
        if name.endswith(s):
            return name[:-len(s)], s
    return name, ""


def match_tensor_role(name: str) -> Tuple[TensorRole, Optional[int], Optional[str], str]:
    """external name -> (role, layer index or None, canonical name or None, suffix kind).

    The suffix kind is ``.weight`` / ``.bias`` / a quantisation companion (``.qweight``, ``.scales`` ...).
    Canonical names carry ``_bias`` for biases and the raw suffix for quantisation companions.
    """
    stem, suffix = split_suffix(name)
    if _NOT_LANGUAGE.search(name):
        return TensorRole.UNKNOWN, None, None, suffix
    m = _LAYER_PREFIX.match(stem)
    if m:
        layer, rest = int(m.group(1)), m.group(2)
        for rx, canon, role in _LAYER_RULES:
            mm = rx.search(rest)
            if mm:
                c = canon
                if "{e}" in c:
                    c = c.replace("{e}", next(g for g in mm.groups() if g and g.isdigit()))
                return role, layer, _with_suffix(f"L{layer}.{c}", suffix), suffix
        return TensorRole.UNKNOWN, layer, None, suffix
    for rx, canon, role in _GLOBAL_RULES:
        if rx.search(stem):
            return role, None, _with_suffix(canon, suffix), suffix
    return TensorRole.UNKNOWN, None, None, suffix


def _with_suffix(canon: str, suffix: str) -> str:
    if suffix in ("", ".weight"):
        return canon
    if suffix in (".bias", "_bias"):
        return canon + "_bias"
    return canon + suffix


def build_name_map(names) -> Dict[str, str]:
    """external -> canonical for every recognised tensor."""
    out = {}
    for n in names:
        _, _, canon, _ = match_tensor_role(n)
        if canon is not None:
            out[n] = canon
    return out
