"""Strategy arbiter: (inference mode x model archetype x hardware) -> strategy bias -> execution plan.

The plan is per client (no globals): it fixes the parallel layout, decode batch cap, prefill chunk, KV precision,
whether the fused collective kernels and CUDA graphs are used, and the overlap policy.

Reference parity: ``InferenceMode{Latency, Throughput}`` x archetype x HW -> ``StrategyBias`` -> ``ExecutionPlan``
(src/engine/arbiter.rs), ``ScenarioHint`` / ``OverlapHint{Auto, PreferOverlap, PreferIsolated, ForceDoubleBuffer,
ForceFlux}`` (src/engine/intent_bias.rs:16-215), graph archetype (src/graph/profile.rs:47-170).
"""
from __future__ import annotations

import enum
from dataclasses import dataclass, field
from typing import Optional

from ..models.config import ModelConfig


class InferenceMode(enum.Enum):
    LATENCY = "latency"
    THROUGHPUT = "throughput"


class ScenarioHint(enum.Enum):
    CHAT = "chat"
    BATCH_OFFLINE = "batch_offline"
    LONG_CONTEXT = "long_context"
    EMBEDDING = "embedding"
    AGENT = "agent"


class OverlapHint(enum.Enum):
    AUTO = "auto"
    PREFER_OVERLAP = "prefer_overlap"
    PREFER_ISOLATED = "prefer_isolated"
    FORCE_DOUBLE_BUFFER = "force_double_buffer"
    FORCE_FLUX = "force_flux"


class Archetype(enum.Enum):
    DENSE_SMALL = "dense_small"        # < 4B params
    DENSE_MEDIUM = "dense_medium"      # 4B - 40B
    DENSE_LARGE = "dense_large"        # > 40B
    MOE = "moe"
    MLA_MOE = "mla_moe"
    ENCODER = "encoder"


def archetype_of(cfg: ModelConfig) -> Archetype:
    if not cfg.causal or cfg.kind in ("embedding", "reranker", "classifier"):
        return Archetype.ENCODER
    if cfg.is_moe:
        return Archetype.MLA_MOE if cfg.is_mla else Archetype.MOE
    p = cfg.param_count()
    return Archetype.DENSE_SMALL if p < 4e9 else Archetype.DENSE_MEDIUM if p < 40e9 else Archetype.DENSE_LARGE


@dataclass
class HardwareSummary:
    gpus: int = 1
    hbm_bytes: int = 180 << 30
    sm_count: int = 148
    nvlink: bool = True
    multimem: bool = True


@dataclass
class StrategyBias:
    batch_weight: float = 0.5        # 0 = minimise latency, 1 = maximise throughput
    memory_weight: float = 0.5       # how hard to squeeze KV
    overlap: OverlapHint = OverlapHint.AUTO
    scenario: ScenarioHint = ScenarioHint.CHAT


@dataclass
class ExecutionPlan:
    tp: int = 1
    pp: int = 1
    ep: int = 1
    max_num_seqs: int = 256
    max_batch_tokens: int = 8192
    prefill_chunk: int = 2048
    kv_dtype: str = "bf16"
    weight_dtype: str = "bf16"
    use_cuda_graphs: bool = True
    fused_collectives: bool = True
    overlap: OverlapHint = OverlapHint.AUTO
    speculative: bool = False
    notes: list = field(default_factory=list)


class StrategyArbiter:
    def __init__(self, hw: HardwareSummary = HardwareSummary()):
        self.hw = hw

    def bias_for(self, mode: InferenceMode, scenario: ScenarioHint = ScenarioHint.CHAT,
                 overlap: OverlapHint = OverlapHint.AUTO) -> StrategyBias:
        b = StrategyBias(scenario=scenario, overlap=overlap)
        b.batch_weight = 0.15 if mode == InferenceMode.LATENCY else 0.9
        if scenario == ScenarioHint.BATCH_OFFLINE:
            b.batch_weight = 1.0
        if scenario == ScenarioHint.LONG_CONTEXT:
            b.memory_weight = 0.9
        if scenario == ScenarioHint.AGENT:
            b.batch_weight = min(b.batch_weight, 0.4)
        return b

    def arbitrate_with_bias(self, cfg: ModelConfig, bias: StrategyBias, dtype_bytes: int = 2) -> ExecutionPlan:
        hw, arch = self.hw, archetype_of(cfg)
        plan = ExecutionPlan(overlap=bias.overlap)
        weight_bytes = cfg.param_count() * dtype_bytes
        usable = hw.hbm_bytes * 0.9
        # parallel layout: smallest TP that leaves >= 30 % of HBM for KV; experts spread when there are any
        tp = 1
        while tp < hw.gpus and (weight_bytes / tp > usable * 0.7 or cfg.num_heads % tp):
            tp *= 2
        if arch in (Archetype.MOE, Archetype.MLA_MOE) and hw.gpus > 1:
            plan.ep = hw.gpus
            tp = 1
            plan.notes.append("experts spread over all GPUs, attention data-parallel")
            if weight_bytes / hw.gpus > usable * 0.8:
                plan.weight_dtype = "fp8"
                plan.notes.append("expert weights do not fit in bf16: block-scaled fp8")
        elif bias.batch_weight < 0.5 and hw.gpus > tp and cfg.num_heads % (tp * 2) == 0 and arch != Archetype.DENSE_SMALL:
            tp = min(hw.gpus, tp * 2)          # latency mode buys speed with more TP
            plan.notes.append("latency mode: extra tensor parallelism")
        plan.tp = tp
        if weight_bytes / (plan.tp * plan.ep) > usable * 0.7 and hw.gpus >= plan.tp * 2 and plan.ep == 1:
            plan.pp = min(hw.gpus // plan.tp, 2)
        plan.max_num_seqs = int(16 + bias.batch_weight * (512 - 16)) if arch != Archetype.ENCODER else 64
        plan.max_batch_tokens = 2048 if bias.batch_weight < 0.5 else 8192
        plan.prefill_chunk = 512 if bias.batch_weight < 0.5 else 2048
        kv_per_seq = cfg.kv_bytes_per_token(plan.tp) * min(cfg.max_position_embeddings, 8192)
        free = usable - weight_bytes / (plan.tp * plan.pp * plan.ep)
        if bias.memory_weight > 0.7 or kv_per_seq * plan.max_num_seqs > free:
            plan.kv_dtype = "fp8"
            plan.notes.append("KV cache in fp8 to fit the batch")
        plan.fused_collectives = hw.nvlink and (plan.tp > 1 or plan.ep > 1)
        if bias.overlap == OverlapHint.PREFER_ISOLATED:
            plan.fused_collectives = False
        plan.speculative = bias.batch_weight < 0.3 and arch != Archetype.ENCODER
        return plan

    def arbitrate(self, cfg: ModelConfig, mode: InferenceMode = InferenceMode.THROUGHPUT, **kw) -> ExecutionPlan:
        return self.arbitrate_with_bias(cfg, self.bias_for(mode, **kw))
