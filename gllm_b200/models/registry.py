"""Model kinds, architecture families and the manifest record.

Reference parity: ``ModelKind{Chat,Embedding,Reranker,Classifier}``, ``ArchFamily``, ``ModelManifest``
(src/manifest/types.rs:151-256); arch alias table (src/arch/registry.rs:12-70, here in ``models/arch.py``).
"""
from __future__ import annotations

import enum
from dataclasses import dataclass, field
from typing import Dict, Optional


class ModelKind(str, enum.Enum):
    CHAT = "chat"
    EMBEDDING = "embedding"
    RERANKER = "reranker"
    CLASSIFIER = "classifier"


class ArchFamily(str, enum.Enum):
    DENSE_DECODER = "dense_decoder"
    MOE_DECODER = "moe_decoder"
    MLA_DECODER = "mla_decoder"
    ENCODER = "encoder"
    VISION = "vision"
    AUDIO = "audio"


def family_of(cfg) -> ArchFamily:
    if not cfg.causal:
        return ArchFamily.ENCODER
    if cfg.is_mla:
        return ArchFamily.MLA_DECODER
    if cfg.is_moe:
        return ArchFamily.MOE_DECODER
    return ArchFamily.DENSE_DECODER


@dataclass
class ModelManifest:
    model_id: str
    kind: ModelKind
    family: ArchFamily
    arch: str
    format: str = ""
    quant: str = ""
    params: int = 0
    extra: Dict[str, str] = field(default_factory=dict)

    @staticmethod
    def from_loaded(model_id: str, loaded, kind: Optional[ModelKind] = None) -> "ModelManifest":
        c = loaded.config
        k = kind or (ModelKind(c.kind) if c.kind in ModelKind._value2member_map_ else ModelKind.CHAT)
        return ModelManifest(model_id, k, family_of(c), c.arch, loaded.format.value, c.quant, c.param_count())
