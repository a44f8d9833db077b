"""Host-side MoE routing tables, capacity, load-balance statistics and hardware dispatch planning.

Reference parity: ``ExpertRouteConfig`` capacity factor -> ``expert_capacity(tokens)``, ``ExpertRouteTable::
from_gate_logits`` with capacity filtering, ``tokens_for_expert``, ``load_balance_loss``, ``topk_with_weights``,
``ExpertLoadBalancer`` hot/cold/hit rates (src/moe/routing.rs:52-452); ``MoeHardwareDispatcher::dispatch`` ->
``MoeDispatchPlan{gpu_experts, cpu_experts}`` hot -> GPU, warm -> CPU (bounded by ``max_cpu_ratio``), cold ->
remote (src/moe/dispatch.rs:26-330); expert heat tracking (src/moe/thermal.rs).
"""
from __future__ import annotations

import math
from collections import deque
from dataclasses import dataclass, field
from typing import Dict, List, Tuple

import torch


@dataclass
class ExpertRouteConfig:
    num_experts: int
    top_k: int
    capacity_factor: float = 1.25
    renormalize: bool = True

    def expert_capacity(self, tokens: int) -> int:
        return max(1, math.ceil(self.capacity_factor * tokens * self.top_k / self.num_experts))


@dataclass
class TokenRoute:
    token: int
    experts: List[int]
    weights: List[float]
    dropped: List[int] = field(default_factory=list)


class ExpertRouteTable:
    def __init__(self, cfg: ExpertRouteConfig, routes: List[TokenRoute]):
        self.cfg, self.routes = cfg, routes

    @staticmethod
    def from_gate_logits(cfg: ExpertRouteConfig, logits: torch.Tensor, enforce_capacity: bool = False):
        probs = torch.softmax(logits.float(), -1)
        w, ids = torch.topk(probs, cfg.top_k, -1)
        if cfg.renormalize:
            w = w / w.sum(-1, keepdim=True)
        cap = cfg.expert_capacity(logits.shape[0])
        load = [0] * cfg.num_experts
        routes = []
        for t in range(logits.shape[0]):
            ex, ws, dropped = [], [], []
            for e, x in zip(ids[t].tolist(), w[t].tolist()):
                if enforce_capacity and load[e] >= cap:
                    dropped.append(e)
                    continue
                load[e] += 1
                ex.append(e)
                ws.append(x)
            routes.append(TokenRoute(t, ex, ws, dropped))
        return ExpertRouteTable(cfg, routes)

    def tokens_for_expert(self, e: int) -> List[Tuple[int, float]]:
        return [(r.token, w) for r in self.routes for x, w in zip(r.experts, r.weights) if x == e]

    def counts(self) -> List[int]:
        c = [0] * self.cfg.num_experts
        for r in self.routes:
            for e in r.experts:
                c[e] += 1
        return c


def load_balance_loss(logits: torch.Tensor, top_k: int) -> float:
    """Switch-style auxiliary loss E * sum_e f_e * P_e (1.0 when perfectly balanced)."""
    probs = torch.softmax(logits.float(), -1)
    E = probs.shape[1]
    _, ids = torch.topk(probs, top_k, -1)
    f = torch.zeros(E).scatter_add_(0, ids.reshape(-1), torch.ones(ids.numel())) / ids.numel()
    return float(E * (f * probs.mean(0)).sum())


class ExpertLoadBalancer:
    """Sliding-window hit statistics; hot = above ``hot_ratio`` x mean, cold = never hit in the window."""

    def __init__(self, num_experts: int, window: int = 64, hot_ratio: float = 2.0):
        self.E, self.window, self.hot_ratio = num_experts, deque(maxlen=window), hot_ratio

    def record(self, counts: List[int]):
        self.window.append(list(counts))

    def totals(self) -> List[int]:
        t = [0] * self.E
        for c in self.window:
            for i, v in enumerate(c):
                t[i] += v
        return t

    def hit_rates(self) -> List[float]:
        t = self.totals()
        s = max(sum(t), 1)
        return [v / s for v in t]

    def hot_experts(self) -> List[int]:
        t = self.totals()
        mean = sum(t) / max(self.E, 1)
        return [i for i, v in enumerate(t) if mean > 0 and v > self.hot_ratio * mean]

    def cold_experts(self) -> List[int]:
        return [i for i, v in enumerate(self.totals()) if v == 0]


@dataclass
class ExpertHardwareAssignment:
    expert_idx: int
    token_count: int


@dataclass
class MoeDispatchPlan:
    gpu_experts: List[ExpertHardwareAssignment]
    cpu_experts: List[ExpertHardwareAssignment]
    remote_experts: List[ExpertHardwareAssignment]


class MoeHardwareDispatcher:
    """Hot experts on the GPU; with weight offloading enabled, warm experts may run on the host (bounded share
    of the tokens) and cold ones are fetched on demand."""

    def __init__(self, resident: List[int], max_cpu_ratio: float = 0.2, cpu_enabled: bool = False):
        self.resident, self.max_cpu_ratio, self.cpu_enabled = set(resident), max_cpu_ratio, cpu_enabled

    def dispatch(self, counts: List[int]) -> MoeDispatchPlan:
        total = max(sum(counts), 1)
        gpu, cpu, remote = [], [], []
        cpu_budget = int(self.max_cpu_ratio * total)
        for e, n in sorted(enumerate(counts), key=lambda x: -x[1]):
            if n == 0:
                continue
            a = ExpertHardwareAssignment(e, n)
            if e in self.resident:
                gpu.append(a)
            elif self.cpu_enabled and n <= cpu_budget:
                cpu.append(a)
                cpu_budget -= n
            else:
                remote.append(a)
        return MoeDispatchPlan(gpu, cpu, remote)


class ExpertThermalTracker:
    """Exponentially decayed heat per expert; drives residency (hot stays in HBM, cold may be paged out)."""

    def __init__(self, num_experts: int, decay: float = 0.95, hot: float = 4.0, cold: float = 0.05):
        self.heat = [0.0] * num_experts
        self.decay, self.hot, self.cold = decay, hot, cold

    def step(self, counts: List[int]):
        for i, c in enumerate(counts):
            self.heat[i] = self.heat[i] * self.decay + c

    def state(self, e: int) -> str:
        h = self.heat[e]
        return "hot" if h >= self.hot else ("cold" if h <= self.cold else "warm")

    def eviction_candidates(self, n: int) -> List[int]:
        return sorted(range(len(self.heat)), key=lambda i: self.heat[i])[:n]
