"""Distributed configuration and rank topology (pure functions of rank / world: unit-testable without GPUs).

Reference parity: ``DistributedConfig{parallel, pd_disagg, kv_distribution, comm, moe}``
(src/engine/distributed_config.rs:118-283) with ``ParallelConfig{tp,pp,ep,cp}`` validated as
``tp * pp * ep == world`` (:167-175), ``KvDistMode`` (:45-52), communication algorithm names and quantised
comm (:810-855, coordinator/comm_schedule.rs:369-486), ``Topology2D/3D`` rank = tp + pp * tp_size
(engine/pipeline/topology.rs:21-205). Here EP re-uses the TP ranks of a stage for expert placement (attention
TP x MoE EP on the same GPUs, as in the benchmark shapes), so the product rule is ``tp * pp * cp == world`` with
``ep`` dividing ``tp * cp``; a stand-alone ``ep`` dimension is also accepted (``tp * pp * ep == world``).
"""
from __future__ import annotations

import enum
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple


class KvDistMode(str, enum.Enum):
    LOCAL = "local"
    ON_DEMAND = "on_demand"
    MIRROR = "mirror"
    PARTIAL_HEAD_MIRROR = "partial_head_mirror"
    TIERED_CACHE = "tiered_cache"


class PdRole(str, enum.Enum):
    COLLOCATED = "collocated"
    PREFILL_ONLY = "prefill_only"
    DECODE_ONLY = "decode_only"


class CommAlgorithm(str, enum.Enum):
    RING = "ring"
    TREE = "tree"
    TOPO_AWARE_RING = "topo_aware_ring"
    CHUNKED_PIPELINE = "chunked_pipeline"
    HIERARCHICAL_RING = "hierarchical_ring"
    HARDWARE_REDUCE = "hardware_reduce"      # NVLS / multimem
    FLUX_PIPELINE = "flux_pipeline"          # GEMM fused with its collective
    COLLNET_DIRECT = "collnet_direct"
    DIRECT = "direct"                        # one-shot peer loads


class CommQuant(str, enum.Enum):
    NONE = "none"
    FP8_E4M3 = "fp8_e4m3"
    FP8_E5M2 = "fp8_e5m2"
    INT8_SYMMETRIC = "int8_symmetric"


class MoePlacement(str, enum.Enum):
    AUTO = "auto"
    ROUND_ROBIN = "round_robin"
    HOT_COLD = "hot_cold"
    CUSTOM = "custom"


class AllToAllMode(str, enum.Enum):
    AUTO = "auto"
    NVLINK = "nvlink"
    RDMA = "rdma"
    HIERARCHICAL = "hierarchical"


class ConfigError(ValueError):
    pass


@dataclass
class ParallelConfig:
    tp: int = 1
    pp: int = 1
    ep: int = 1
    cp: int = 1
    ep_shares_tp: bool = True   # experts are spread over the TP(xCP) ranks of a stage

    def world_size(self) -> int:
        return self.tp * self.pp * self.cp * (1 if self.ep_shares_tp else self.ep)

    def validate(self, world: int):
        for n, v in (("tp", self.tp), ("pp", self.pp), ("ep", self.ep), ("cp", self.cp)):
            if v < 1:
                raise ConfigError(f"{n} must be >= 1")
        if self.world_size() != world:
            raise ConfigError(f"tp*pp*cp{'' if self.ep_shares_tp else '*ep'} = {self.world_size()} != world size {world}")
        if self.ep_shares_tp and (self.tp * self.cp) % self.ep:
            raise ConfigError(f"ep={self.ep} must divide tp*cp={self.tp * self.cp}")


@dataclass
class CommConfig:
    algorithm: CommAlgorithm = CommAlgorithm.FLUX_PIPELINE
    quant: CommQuant = CommQuant.NONE
    timeout_s: float = 30.0
    overlap: str = "auto"         # auto | prefer_overlap | prefer_isolated | force_double_buffer | force_flux
    comm_sm_ratio: float = 0.3


@dataclass
class MoeDistConfig:
    placement: MoePlacement = MoePlacement.AUTO
    all_to_all: AllToAllMode = AllToAllMode.AUTO
    custom_map: Optional[Dict[int, int]] = None
    hot_experts: List[int] = field(default_factory=list)
    eplb_window_s: float = 60.0
    eplb_threshold: float = 2.0


@dataclass
class DistributedConfig:
    parallel: ParallelConfig = field(default_factory=ParallelConfig)
    pd_role: PdRole = PdRole.COLLOCATED
    kv_distribution: KvDistMode = KvDistMode.LOCAL
    comm: CommConfig = field(default_factory=CommConfig)
    moe: MoeDistConfig = field(default_factory=MoeDistConfig)

    def validate(self, world: int):
        self.parallel.validate(world)
        if self.pd_role != PdRole.COLLOCATED and world < 2:
            raise ConfigError("prefill/decode disaggregation needs at least two ranks")


@dataclass(frozen=True)
class RankCoord:
    rank: int
    tp: int
    cp: int
    pp: int
    ep: int


class Topology:
    """rank = tp_rank + tp * (cp_rank + cp * pp_rank): TP innermost (NVLink neighbours), PP outermost."""

    def __init__(self, cfg: ParallelConfig, world: int):
        cfg.validate(world)
        self.cfg, self.world = cfg, world

    def coord(self, rank: int) -> RankCoord:
        c = self.cfg
        tp = rank % c.tp
        cp = (rank // c.tp) % c.cp
        pp = rank // (c.tp * c.cp) if c.ep_shares_tp else (rank // (c.tp * c.cp)) % c.pp
        stage_rank = rank % (c.tp * c.cp)
        ep = stage_rank % c.ep if c.ep_shares_tp else rank // (c.tp * c.cp * c.pp)
        return RankCoord(rank, tp, cp, pp, ep)

    def rank_of(self, tp: int, cp: int = 0, pp: int = 0) -> int:
        return tp + self.cfg.tp * (cp + self.cfg.cp * pp)

    def tp_group(self, rank: int) -> List[int]:
        c = self.coord(rank)
        return [self.rank_of(t, c.cp, c.pp) for t in range(self.cfg.tp)]

    def cp_group(self, rank: int) -> List[int]:
        c = self.coord(rank)
        return [self.rank_of(c.tp, k, c.pp) for k in range(self.cfg.cp)]

    def pp_group(self, rank: int) -> List[int]:
        c = self.coord(rank)
        return [self.rank_of(c.tp, c.cp, p) for p in range(self.cfg.pp)]

    def ep_group(self, rank: int) -> List[int]:
        """Ranks that together hold one copy of every expert."""
        c = self.coord(rank)
        base = self.rank_of(0, 0, c.pp)
        stage = list(range(base, base + self.cfg.tp * self.cfg.cp))
        block = (rank - base) // self.cfg.ep * self.cfg.ep
        return stage[block:block + self.cfg.ep]

    def pp_next(self, rank: int) -> Optional[int]:
        c = self.coord(rank)
        return None if c.pp + 1 >= self.cfg.pp else self.rank_of(c.tp, c.cp, c.pp + 1)

    def pp_prev(self, rank: int) -> Optional[int]:
        c = self.coord(rank)
        return None if c.pp == 0 else self.rank_of(c.tp, c.cp, c.pp - 1)

    def is_tp_master(self, rank: int) -> bool:
        return self.coord(rank).tp == 0

    def all_groups(self, kind: str) -> List[List[int]]:
        fn = {"tp": self.tp_group, "cp": self.cp_group, "pp": self.pp_group, "ep": self.ep_group}[kind]
        seen, out = set(), []
        for r in range(self.world):
            g = tuple(fn(r))
            if g not in seen:
                seen.add(g)
                out.append(list(g))
        return out


def select_algorithm(nbytes: int, world: int, has_nvls: bool, fused_with_gemm: bool) -> CommAlgorithm:
    """All-reduce algorithm choice on one NVSwitch node (the reference selects by topology and message size)."""
    if fused_with_gemm:
        return CommAlgorithm.FLUX_PIPELINE
    if has_nvls and nbytes >= 64 * 1024:
        return CommAlgorithm.HARDWARE_REDUCE
    if nbytes < 256 * 1024:
        return CommAlgorithm.DIRECT
    return CommAlgorithm.RING if world > 2 else CommAlgorithm.DIRECT
