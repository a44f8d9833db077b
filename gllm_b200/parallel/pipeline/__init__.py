"""Pipeline parallelism for inference: stage <-> layer ranges, micro-batch schedules, activation transport over
NCCL point-to-point on a side stream, bubble analysis, and heartbeat-based stage fault recovery.

Reference parity (src/engine/pipeline/*): ``PipelineConfig`` stage/layer ranges (config.rs:23-190), PP weight
filter (loader/weight_shard.rs:184-305), ``MicroBatchScheduler`` split (micro_batch.rs:64-130), GPipe / 1F1B /
interleaved-with-virtual-stages / zero-bubble op lists with warm-up / steady / cool-down phases
(scheduler.rs:135-375, interleaved.rs), bubble analyser and adaptive micro-batch sizer, ``ActivationTransport``
send/recv of ``micro_batch x hidden`` with optional FP8 / INT8 activation quantisation (activation_xfer.rs:151-
560), per-stage KV manager (scheduler.rs:884-1080), ``StageFaultRecovery`` heartbeat table, isolation and
migration plan driven by caller-supplied clocks (fault_recovery.rs:19-550). The reference's schedules speak a
training vocabulary (forward + backward); an inference engine only has forward ops, so the backward entries of
1F1B / zero-bubble exist for parity of the planner and are filtered by ``forward_only``. Gradient sync is out
of scope.
"""
from __future__ import annotations

import enum
import math
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import torch


# ------------------------------------------------------------------------------------------------
# stage layout
# ------------------------------------------------------------------------------------------------
@dataclass
class PipelineConfig:
    num_layers: int
    num_stages: int
    virtual_stages: int = 1            # interleaved schedule: chunks of layers per rank
    layer_costs: Optional[List[float]] = None   # relative cost per layer (embedding / head can be folded in)

    def stage_ranges(self) -> List[range]:
        """Contiguous layer ranges, balanced by cost (equal cost -> remainder spread over the first stages)."""
        n = self.num_stages * self.virtual_stages
        if n > self.num_layers:
            raise ValueError(f"{n} pipeline chunks for {self.num_layers} layers")
        if self.layer_costs is None:
            base, rem = divmod(self.num_layers, n)
            out, s = [], 0
            for i in range(n):
                e = s + base + (1 if i < rem else 0)
                out.append(range(s, e))
                s = e
            return out
        total = sum(self.layer_costs)
        out, s, acc = [], 0, 0.0
        for i in range(n):
            target = total * (i + 1) / n
            e = s
            while e < self.num_layers - (n - 1 - i) and (acc + self.layer_costs[e] <= target or e == s):
                acc += self.layer_costs[e]
                e += 1
            out.append(range(s, e))
            s = e
        out[-1] = range(out[-1].start, self.num_layers)
        return out

    def layers_of_stage(self, stage: int) -> List[range]:
        """With interleaving, stage s owns chunks s, s + num_stages, s + 2*num_stages ..."""
        r = self.stage_ranges()
        return [r[stage + v * self.num_stages] for v in range(self.virtual_stages)]

    def stage_of_layer(self, layer: int) -> int:
        for i, r in enumerate(self.stage_ranges()):
            if layer in r:
                return i % self.num_stages
        raise IndexError(layer)


def pp_weight_filter(name: str, layers: range, is_first: bool, is_last: bool, tied: bool = False) -> bool:
    """Does this pipeline stage need the canonical tensor ``name``?"""
    if name.startswith("L"):
        return int(name[1:].split(".", 1)[0]) in layers
    if name in ("embed_tokens", "position_embeddings", "token_type_embeddings", "embed_norm", "embed_norm_bias"):
        return is_first or (tied and is_last and name == "embed_tokens")
    if name in ("final_norm", "lm_head", "classifier", "pooler"):
        return is_last
    return True


# ------------------------------------------------------------------------------------------------
# micro-batches and schedules
# ------------------------------------------------------------------------------------------------
def split_micro_batches(total: int, num_micro: int) -> List[Tuple[int, int]]:
    """(start, size) per micro-batch, sizes differing by at most one."""
    num_micro = max(1, min(num_micro, total))
    base, rem = divmod(total, num_micro)
    out, s = [], 0
    for i in range(num_micro):
        n = base + (1 if i < rem else 0)
        out.append((s, n))
        s += n
    return out


class OpKind(str, enum.Enum):
    FORWARD = "F"
    BACKWARD = "B"
    BACKWARD_WEIGHT = "W"
    RECV = "recv"
    SEND = "send"


@dataclass(frozen=True)
class PipeOp:
    kind: OpKind
    micro: int
    chunk: int = 0       # virtual stage index
    phase: str = "steady"


def gpipe_schedule(stage: int, stages: int, micros: int, forward_only: bool = True) -> List[PipeOp]:
    ops = [PipeOp(OpKind.FORWARD, m, 0, "warmup" if m < stages - stage - 1 else "steady") for m in range(micros)]
    if not forward_only:
        ops += [PipeOp(OpKind.BACKWARD, m, 0, "cooldown") for m in reversed(range(micros))]
    return ops


def one_f_one_b_schedule(stage: int, stages: int, micros: int, forward_only: bool = False) -> List[PipeOp]:
    warm = min(stages - stage - 1, micros)
    ops = [PipeOp(OpKind.FORWARD, m, 0, "warmup") for m in range(warm)]
    f, b = warm, 0
    while f < micros:
        ops.append(PipeOp(OpKind.FORWARD, f, 0, "steady"))
        f += 1
        ops.append(PipeOp(OpKind.BACKWARD, b, 0, "steady"))
        b += 1
    while b < micros:
        ops.append(PipeOp(OpKind.BACKWARD, b, 0, "cooldown"))
        b += 1
    return [o for o in ops if not forward_only or o.kind == OpKind.FORWARD]


def interleaved_schedule(stage: int, stages: int, micros: int, virtual: int, forward_only: bool = True) -> List[PipeOp]:
    """Interleaved 1F1B (virtual stages): micro-batches advance in groups of ``stages`` through each chunk."""
    if micros % stages:
        raise ValueError("interleaved schedule needs micro-batches divisible by the number of stages")
    total = micros * virtual
    fwd = []
    for i in range(total):
        group, within = divmod(i, stages * virtual)
        chunk, pos = divmod(within, stages)
        fwd.append((group * stages + pos, chunk))
    warm = min((stages - stage - 1) * 2 + (virtual - 1) * stages, total)
    ops = [PipeOp(OpKind.FORWARD, m, c, "warmup" if i < warm else "steady") for i, (m, c) in enumerate(fwd)]
    if not forward_only:
        ops += [PipeOp(OpKind.BACKWARD, m, virtual - 1 - c, "cooldown") for (m, c) in fwd]
    return ops


def zero_bubble_schedule(stage: int, stages: int, micros: int) -> List[PipeOp]:
    """ZB-H1: backward split into input-gradient (B) and weight-gradient (W); W fills the cool-down bubble."""
    ops = one_f_one_b_schedule(stage, stages, micros)
    out, pending_w = [], []
    for o in ops:
        out.append(o)
        if o.kind == OpKind.BACKWARD:
            pending_w.append(o.micro)
            if o.phase == "cooldown" and pending_w:
                out.append(PipeOp(OpKind.BACKWARD_WEIGHT, pending_w.pop(0), 0, "cooldown"))
    out += [PipeOp(OpKind.BACKWARD_WEIGHT, m, 0, "cooldown") for m in pending_w]
    return out


def bubble_fraction(stages: int, micros: int, virtual: int = 1) -> float:
    """Idle share of a forward-only pipeline: (p - 1) / (v*m + p - 1)."""
    return (stages - 1) / (virtual * micros + stages - 1)


def choose_micro_batches(batch_tokens: int, stages: int, target_bubble: float = 0.05, min_tokens: int = 256,
                         max_micro: int = 64) -> int:
    """Smallest micro-batch count that meets the bubble target without starving the tensor cores."""
    best = 1
    for m in range(1, max_micro + 1):
        if batch_tokens // m < min_tokens and m > 1:
            break
        best = m
        if bubble_fraction(stages, m) <= target_bubble:
            break
    return best


# ------------------------------------------------------------------------------------------------
# activation transport (NCCL p2p on a side stream, bf16 by default)
# ------------------------------------------------------------------------------------------------
class ActivationTransport:
    def __init__(self, comm, prev_rank: Optional[int], next_rank: Optional[int], hidden: int, device, dtype=torch.bfloat16,
                 quant: str = "none", max_tokens: int = 8192):
        self.comm, self.prev, self.next = comm, prev_rank, next_rank
        self.hidden, self.device, self.dtype, self.quant = hidden, torch.device(device), dtype, quant
        self.stream = torch.cuda.Stream(device=self.device) if self.device.type == "cuda" else None
        wire = torch.float8_e4m3fn if quant == "fp8" else (torch.int8 if quant == "int8" else dtype)
        self._recv_buf = torch.empty((max_tokens, hidden), dtype=wire, device=self.device)
        self._scale_buf = torch.empty((max_tokens, 1), dtype=torch.float32, device=self.device)
        self.bytes_sent = 0

    def _pack(self, x):
        if self.quant == "none":
            return x.to(self.dtype).contiguous(), None
        amax = x.float().abs().amax(-1, keepdim=True).clamp_min(1e-12)
        if self.quant == "fp8":
            s = amax / 448.0
            return (x.float() / s).to(torch.float8_e4m3fn), s
        s = amax / 127.0
        return torch.clamp((x.float() / s).round(), -127, 127).to(torch.int8), s

    def _unpack(self, q, s):
        return q.to(self.dtype) if s is None else (q.float() * s).to(self.dtype)

    def send(self, x: torch.Tensor, async_op: bool = True):
        """Stage i -> i+1. Returns a list of work handles (empty on the last stage)."""
        if self.next is None:
            return []
        q, s = self._pack(x)
        works = []
        ctx = torch.cuda.stream(self.stream) if self.stream is not None else _null()
        if self.stream is not None:
            self.stream.wait_stream(torch.cuda.current_stream(self.device))
        with ctx:
            payload = q.view(torch.uint8) if q.dtype == torch.float8_e4m3fn else q
            works.append(self.comm.send(payload, self.next, async_op=async_op))
            if s is not None:
                works.append(self.comm.send(s, self.next, async_op=async_op))
        self.bytes_sent += q.numel() * q.element_size()
        return [w for w in works if w is not None]

    def recv(self, tokens: int) -> torch.Tensor:
        if self.prev is None:
            raise RuntimeError("first stage has nothing to receive")
        buf = self._recv_buf[:tokens]
        payload = buf.view(torch.uint8) if buf.dtype == torch.float8_e4m3fn else buf
        self.comm.recv(payload, self.prev)
        s = None
        if self.quant != "none":
            s = self._scale_buf[:tokens]
            self.comm.recv(s, self.prev)
        return self._unpack(buf, s)


class _null:
    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False


# ------------------------------------------------------------------------------------------------
# overlap model and SM partition hint
# ------------------------------------------------------------------------------------------------
def overlap_model(compute_ms: float, comm_ms: float, mode: str = "auto", comm_sm_ratio: float = 0.3) -> Dict[str, float]:
    """Estimated step time when communication runs beside compute on a slice of the SMs."""
    if mode in ("prefer_isolated", "serial"):
        return {"step_ms": compute_ms + comm_ms, "exposed_comm_ms": comm_ms, "comm_sm_ratio": 0.0}
    slowed = compute_ms / max(1e-9, 1.0 - comm_sm_ratio)
    exposed = max(0.0, comm_ms - slowed)
    return {"step_ms": slowed + exposed, "exposed_comm_ms": exposed, "comm_sm_ratio": comm_sm_ratio}


# ------------------------------------------------------------------------------------------------
# per-stage KV accounting
# ------------------------------------------------------------------------------------------------
@dataclass
class StageKvManager:
    stage: int
    layers: range
    kv_bytes_per_token_layer: int
    budget_bytes: int
    used_tokens: int = 0

    def capacity_tokens(self) -> int:
        per = self.kv_bytes_per_token_layer * max(len(self.layers), 1)
        return self.budget_bytes // max(per, 1)

    def reserve(self, tokens: int) -> bool:
        if self.used_tokens + tokens > self.capacity_tokens():
            return False
        self.used_tokens += tokens
        return True

    def release(self, tokens: int):
        self.used_tokens = max(0, self.used_tokens - tokens)


# ------------------------------------------------------------------------------------------------
# stage fault recovery (host logic, caller supplies the clock)
# ------------------------------------------------------------------------------------------------
class StageStatus(str, enum.Enum):
    HEALTHY = "healthy"
    SUSPECT = "suspect"
    FAULTED = "faulted"
    ISOLATED = "isolated"


@dataclass
class HeartbeatConfig:
    interval_s: float = 1.0
    timeout_s: float = 5.0
    max_consecutive_misses: int = 3


@dataclass
class MigrationPlan:
    faulted_stage: int
    target_stage: int
    layers: List[int]
    weight_bytes: int
    kv_bytes: int
    parallel: bool
    estimated_s: float


class StageFaultRecovery:
    def __init__(self, num_stages: int, cfg: HeartbeatConfig = None):
        self.cfg = cfg or HeartbeatConfig()
        self.last_seen: Dict[int, float] = {s: 0.0 for s in range(num_stages)}
        self.misses: Dict[int, int] = {s: 0 for s in range(num_stages)}
        self.status: Dict[int, StageStatus] = {s: StageStatus.HEALTHY for s in range(num_stages)}

    def heartbeat(self, stage: int, now: float):
        if self.status[stage] == StageStatus.ISOLATED:
            return
        self.last_seen[stage] = now
        self.misses[stage] = 0
        self.status[stage] = StageStatus.HEALTHY

    def detect(self, now: float) -> Dict[int, StageStatus]:
        for s, seen in self.last_seen.items():
            if self.status[s] == StageStatus.ISOLATED:
                continue
            late = now - seen
            if late > self.cfg.timeout_s:
                self.misses[s] = max(self.misses[s], int(late // self.cfg.interval_s))
                self.status[s] = (StageStatus.FAULTED if self.misses[s] >= self.cfg.max_consecutive_misses
                                  else StageStatus.SUSPECT)
            elif late > self.cfg.interval_s * 2:
                self.status[s] = StageStatus.SUSPECT
        return dict(self.status)

    def isolate(self, stage: int):
        self.status[stage] = StageStatus.ISOLATED

    def plan_migration(self, stage: int, pcfg: PipelineConfig, bytes_per_layer: int, kv_bytes: int,
                       link_gbs: float = 700.0, parallel: bool = True) -> MigrationPlan:
        """Move the faulted stage's layers to the neighbour with the fewest layers."""
        ranges = pcfg.stage_ranges()
        healthy = [s for s, st in self.status.items() if st == StageStatus.HEALTHY and s != stage]
        if not healthy:
            raise RuntimeError("no healthy stage left to migrate to")
        target = min(healthy, key=lambda s: (len(ranges[s]), abs(s - stage)))
        layers = list(ranges[stage])
        wbytes = bytes_per_layer * len(layers)
        secs = (max(wbytes, kv_bytes) if parallel else wbytes + kv_bytes) / (link_gbs * 1e9)
        return MigrationPlan(stage, target, layers, wbytes, kv_bytes, parallel, secs)

    @staticmethod
    def verify_post_migration_equivalence(before: Dict[int, List[int]], after: Dict[int, List[int]]) -> bool:
        """Every layer is still owned exactly once and in order."""
        flat = lambda d: sorted(l for ls in d.values() for l in ls)
        return flat(before) == flat(after) and all(ls == sorted(ls) for ls in after.values())
