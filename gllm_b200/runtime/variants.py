"""Registry of compiled kernel variants and the dispatch-time choice among them.

The reference keys JIT-compiled mega-kernel variants by mechanism and checks an instruction-cache budget; here a
variant is a captured CUDA graph / kernel configuration (tile shape, split count, fused or not) with a measured
cost, and the budget is device memory held by captured graphs.

Reference parity: ``VariantKey`` / ``CompiledVariant`` / ``MechanismId`` / ``CodeSection``, the <= 80 % budget
check (``L1iBudgetExceeded``) and ``select_variant_for_batch`` (src/jit/variant_registry.rs:20-190;
src/engine/mega_kernel/executor_ops.inc.rs:1317).
"""
from __future__ import annotations

import enum
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple


class MechanismId(enum.Enum):
    DENSE = "dense"
    KIVI_QUANT = "kivi_quant"
    GUARDRAIL_PROBE = "guardrail_probe"
    EARLY_EXIT = "early_exit"
    SPECULATIVE = "speculative"
    MOE_EP = "moe_ep"
    SAMPLED = "sampled"          # non-greedy sampling in the graph


class CodeSection(enum.Enum):
    HOT = "hot"
    WARM = "warm"
    COLD = "cold"


@dataclass(frozen=True)
class VariantKey:
    bucket: int
    mechanisms: Tuple[MechanismId, ...] = (MechanismId.DENSE,)


@dataclass
class CompiledVariant:
    key: VariantKey
    handle: Any                  # CUDA graph or callable
    bytes: int = 0
    section: CodeSection = CodeSection.HOT
    hits: int = 0
    us: float = 0.0


class BudgetExceeded(RuntimeError):
    pass


class VariantRegistry:
    def __init__(self, budget_bytes: int, max_fill: float = 0.8):
        self.budget, self.max_fill = budget_bytes, max_fill
        self.variants: Dict[VariantKey, CompiledVariant] = {}

    def used(self) -> int:
        return sum(v.bytes for v in self.variants.values())

    def register(self, v: CompiledVariant, evict: bool = True):
        limit = self.budget * self.max_fill
        while self.used() + v.bytes > limit:
            cold = sorted((x for x in self.variants.values() if x.section != CodeSection.HOT or x.hits == 0), key=lambda x: x.hits)
            if not evict or not cold:
                raise BudgetExceeded(f"variant {v.key} needs {v.bytes} bytes; {self.used()} of {int(limit)} in use")
            self.variants.pop(cold[0].key)
        self.variants[v.key] = v

    def select_for_batch(self, batch: int, mechanisms: Tuple[MechanismId, ...] = (MechanismId.DENSE,)) -> Optional[CompiledVariant]:
        """Smallest registered bucket >= batch with exactly the requested mechanisms."""
        fits = [v for k, v in self.variants.items() if k.mechanisms == tuple(mechanisms) and k.bucket >= batch]
        if not fits:
            return None
        best = min(fits, key=lambda v: v.key.bucket)
        best.hits += 1
        return best

    def reclassify(self):
        total = sum(v.hits for v in self.variants.values()) or 1
        for v in self.variants.values():
            share = v.hits / total
            v.section = CodeSection.HOT if share > 0.2 else CodeSection.WARM if share > 0.02 else CodeSection.COLD
