"""The engine's responsibilities under the names the reference uses for its six coordinators
(src/engine/executor.rs:27-35; src/engine/coordinator/*): thin views over ``LLMEngine`` so that code written against
that vocabulary finds the same seams here.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional

from ..parallel.config import KvDistMode, PdRole
from ..parallel.pd import kv_dist_plan, resolve_pd_role
from ..scheduler.observer import BasicObserver


class DispatchCoordinator:
    """Scheduler + batcher + requests + policy, and the prefill / decode role of this rank."""

    def __init__(self, engine, pd_role: PdRole = PdRole.COLLOCATED):
        self.engine, self.pd_role = engine, pd_role

    def enqueue(self, prompt_ids, **kw) -> int:
        return self.engine.add_request(prompt_ids, **kw)

    def phases(self) -> Dict[str, bool]:
        b = self.engine.batcher
        return resolve_pd_role(self.pd_role, b.num_waiting > 0, b.num_running > 0)

    def queue_depths(self):
        b = self.engine.batcher
        return {"waiting": b.num_waiting, "running": b.num_running}


class KvCoordinator:
    """The paged pool, its distribution mode and the optional swap tier."""

    def __init__(self, engine, mode: KvDistMode = KvDistMode.LOCAL, swap=None, rank: int = 0, world: int = 1):
        self.engine, self.mode, self.swap, self.rank, self.world = engine, mode, swap, rank, world

    def plan(self):
        return kv_dist_plan(self.mode, self.rank, self.world, self.engine.mc.num_kv_heads)

    def occupancy(self) -> float:
        b = self.engine.batcher
        return 1.0 - b.num_free_pages / max(b.num_total_pages, 1)

    @property
    def memory(self):
        """The three-tier page accounting (``GlobalMemoryManager``) over this engine's pools: HBM pages of the batcher,
        pinned host pages and NVMe slots of the swap tier. Occupancy is refreshed from the pools on every call."""
        from ..scheduler.memory_manager import GlobalMemoryManager
        from ..scheduler.types import Tier
        b = self.engine.batcher
        sw = self.swap
        host = int(sw.host_pool.shape[0]) if sw is not None else 0
        nvme = (len(sw.nvme.free) + sum(1 for r in sw.records.values() if int(r.tier) == 2)) if (
            sw is not None and sw.nvme is not None) else 0
        if getattr(self, "_mem", None) is None or self._mem.cap[Tier.L1_GPU] != b.num_total_pages:
            self._mem = GlobalMemoryManager(b.num_total_pages, host, nvme)
        m = self._mem
        m.used[Tier.L1_GPU] = b.num_total_pages - b.num_free_pages
        if sw is not None:
            m.used[Tier.L2_CPU] = host - len(sw.host_free)
            m.used[Tier.L3_NVME] = nvme - len(sw.nvme.free) if sw.nvme is not None else 0
        return m

    def plan_prefill(self, prompt_tokens: int):
        """Whether a prompt's pages fit the free HBM pages now (``fully_resident``) or the prefill has to run chunk by
        chunk with part of its pages waiting in the host tier (``pipelined``)."""
        return self.memory.plan_prefill(prompt_tokens, chunk_tokens=self.engine.cfg.prefill_chunk)

    def reclaim(self, pages: int) -> int:
        """Ask the swap tier (when there is one) to make room."""
        if self.swap is None:
            return 0
        return len(self.swap.eviction_pass(hbm_used_ratio=1.0)[:pages])


class ComputeCoordinator:
    """Tensor-parallel context of the model and which collective path it takes."""

    def __init__(self, engine):
        self.engine = engine

    def tp_mode(self) -> str:
        tp = self.engine.model.tp
        return "none" if tp is None else (tp.mode + ("+multimem" if getattr(tp, "uses_multimem", False) else ""))


class InferenceCoordinator:
    def __init__(self, engine):
        self.engine = engine

    def step(self):
        return self.engine.step()

    def drain(self):
        return self.engine.run_until_done()


class ModelContextHolder:
    def __init__(self, engine):
        self.model, self.config, self.tokenizer = engine.model, engine.mc, engine.tokenizer


class ObservabilityCoordinator:
    """Captures a ``SystemState`` every step and feeds it back to the scheduler policy."""

    def __init__(self, engine):
        self.engine, self.observer = engine, BasicObserver()
        self.eplb = None              # moe.eplb.Eplb of an MoE model: sliding window of per-expert token counts
        self.eplb_state: Dict[str, object] = {}

    def capture(self):
        b = self.engine.batcher
        st = self.observer.system_state(free_pages=b.num_free_pages, total_pages=b.num_total_pages,
                                        fragmentation=b.fragmentation, running=b.num_running, waiting=b.num_waiting)
        b.set_system_state(st)
        self.capture_expert_load()
        return st

    def capture_expert_load(self, reduce: bool = False):
        """Expert-load sample for the load balancer: the most recent routing decision of the model's MoE layers goes
        into the sliding window; the window's totals give the imbalance (max / mean) and, beyond the threshold, the
        hot experts a HotCold placement would mirror. The step loop samples this rank's own routing only;
        ``reduce=True`` sums the windows over the expert-parallel ranks first and is a collective: every rank of the
        group has to make the call (e.g. from the serving loop's periodic maintenance point).
        Reference: EPLB window, cross-rank reduction and decision (src/moe/eplb.rs:18-243)."""
        model = self.engine.model
        cfg = getattr(model, "cfg", None)
        if cfg is None or not getattr(cfg, "is_moe", False):
            return None
        holder = getattr(model, "__dict__", {}).get("_moe_ws") or {}
        ids = next((ws.last_ids for ws in holder.values() if getattr(ws, "last_ids", None) is not None), None)
        if ids is None:
            return None
        import torch
        from ..moe.eplb import Eplb
        from ..parallel.config import MoeDistConfig
        if self.eplb is None:
            self.eplb = Eplb(cfg.num_experts)
        counts = torch.bincount(ids.reshape(-1).long().clamp_(0, cfg.num_experts - 1), minlength=cfg.num_experts)
        self.eplb.record(counts)
        totals = self.eplb.local_totals()
        ep = getattr(model, "ep", None)
        group = getattr(ep, "group", None)
        if reduce and ep is not None and getattr(ep, "size", 1) > 1:
            import torch.distributed as dist
            t = totals.to(ids.device)
            dist.all_reduce(t, group=group)
            totals = t.cpu()
        dist_cfg = MoeDistConfig()
        decision = self.eplb.decide(totals, dist_cfg)
        self.eplb_state = {"imbalance": self.eplb.imbalance(totals), "totals": totals,
                           "hot_experts": list(decision.hot_experts) if decision is not None else [],
                           "placement": decision.placement if decision is not None else dist_cfg.placement}
        return self.eplb_state


@dataclass
class Coordinators:
    dispatch: DispatchCoordinator
    kv: KvCoordinator
    compute: ComputeCoordinator
    inference: InferenceCoordinator
    model_ctx: ModelContextHolder
    observability: ObservabilityCoordinator

    @staticmethod
    def of(engine, **kw) -> "Coordinators":
        return Coordinators(DispatchCoordinator(engine, kw.get("pd_role", PdRole.COLLOCATED)),
                            KvCoordinator(engine, kw.get("kv_mode", KvDistMode.LOCAL), kw.get("swap")),
                            ComputeCoordinator(engine), InferenceCoordinator(engine), ModelContextHolder(engine),
                            ObservabilityCoordinator(engine))
