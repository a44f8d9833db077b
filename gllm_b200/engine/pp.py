"""Pipeline parallelism inside the serving engine.

Every stage runs a full ``LLMEngine`` over ITS layers (``DecoderModel(layers=...)``) and its slice of the KV cache,
with the SAME request stream and therefore the same scheduler decisions (the C++ batcher is deterministic). In a
step, stage s receives the hidden states of the step's tokens from stage s - 1 (NCCL / gloo p2p), runs its layers,
and sends them on; the last stage samples and the sampled tokens are broadcast to every stage of the pipeline, so all
batchers commit the same tokens. With tensor parallelism inside a stage, rank (stage s, tp i) talks to rank
(stage s + 1, tp i): activations are replicated inside a TP group.

Reference parity: stage <-> layer ranges and topology (src/engine/pipeline/config.rs:23-190,
src/engine/pipeline/topology.rs:21-205: rank = tp + pp * tp_size, TP-master-only send in the reference, every TP
rank its own lane here), ``ActivationTransport`` (src/engine/pipeline/activation_xfer.rs:151-560), the executor
step that wires it (src/engine/executor_step.rs:859-973).
"""
from __future__ import annotations

from typing import Optional

import torch


class PipelineContext:
    def __init__(self, comm, stage: int, num_stages: int, *, tp_size: int = 1, tp_index: int = 0, pp_group=None):
        """``comm``: world ``CommHandle``; ``pp_group``: handle over the ranks {stage * tp_size + tp_index} of this
        pipeline lane (None: the world is one lane)."""
        self.comm, self.stage, self.num_stages = comm, stage, num_stages
        self.tp_size, self.tp_index = tp_size, tp_index
        self.lane = pp_group or comm
        rank_of = lambda s: s * tp_size + tp_index
        self.prev = None if stage == 0 else rank_of(stage - 1)
        self.next = None if stage == num_stages - 1 else rank_of(stage + 1)
        self.last_rank = rank_of(num_stages - 1)
        self.stats = {"sent_bytes": 0, "recv_bytes": 0}

    @property
    def is_first(self) -> bool:
        return self.stage == 0

    @property
    def is_last(self) -> bool:
        return self.stage == self.num_stages - 1

    def recv_hidden(self, buf: torch.Tensor) -> torch.Tensor:
        self.comm.recv(buf, self.prev)
        self.stats["recv_bytes"] += buf.numel() * buf.element_size()
        return buf

    def send_hidden(self, x: torch.Tensor):
        self.comm.send(x.contiguous(), self.next)
        self.stats["sent_bytes"] += x.numel() * x.element_size()

    def share_tokens(self, tok: torch.Tensor) -> torch.Tensor:
        """The last stage's sampled tokens reach every stage of this lane (in place)."""
        import torch.distributed as dist
        if self.num_stages > 1:
            dist.broadcast(tok, src=self.last_rank, group=self.lane.group)
        return tok


def build_pipeline(comm, *, pp: int, tp: int = 1) -> PipelineContext:
    """Rank layout: rank = stage * tp + tp_index. Every rank of the world must call this (sub-groups are collective)."""
    stage, tpi = comm.rank // tp, comm.rank % tp
    lane = None
    if tp > 1:
        for i in range(tp):      # every rank takes part in creating every lane's group
            g = comm.subgroup([s * tp + i for s in range(pp)])
            if i == tpi:
                lane = g
    return PipelineContext(comm, stage, pp, tp_size=tp, tp_index=tpi, pp_group=lane)
