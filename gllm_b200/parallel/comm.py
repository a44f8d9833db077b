"""Communication handle over ``torch.distributed`` (NCCL on GPUs, gloo on CPU): device tensors in their own
dtype, collectives return work handles, bootstrap by the launcher's rendezvous.

Reference parity: ``CommHandleWrapper{rank, world_size, inner}`` with ``all_reduce / reduce_scatter / all_gather /
broadcast / send / recv`` (+ ``_async`` futures), ``new_for_test(rank, world)`` without a backend, collectives on
an uninitialised handle return an error, ``destroy()`` = barrier then drop, ``set_timeout``
(src/engine/distributed_config.rs:300-855). Differences by design: no host f32 staging, counts travel as
integers, and every rank shares the launcher's rendezvous instead of generating its own unique id
(the reference's ``init_nccl`` pitfall, :347-357).
"""
from __future__ import annotations

import datetime
from typing import List, Optional

import torch


class CommError(RuntimeError):
    pass


class CommHandle:
    def __init__(self, rank: int, world_size: int, group=None, initialized: bool = False):
        self.rank, self.world_size, self.group, self._init = rank, world_size, group, initialized
        self.timeout_s = 30.0

    # ---- construction ---------------------------------------------------------------------------
    @staticmethod
    def new_for_test(rank: int, world_size: int) -> "CommHandle":
        """A handle with rank arithmetic but no backend: every collective raises ``CommError``."""
        return CommHandle(rank, world_size, None, False)

    @staticmethod
    def from_env(backend: Optional[str] = None, device=None, timeout_s: float = 30.0) -> "CommHandle":
        import torch.distributed as dist
        if not dist.is_initialized():
            be = backend or ("nccl" if torch.cuda.is_available() else "gloo")
            kw = {"device_id": device} if (be == "nccl" and device is not None) else {}
            dist.init_process_group(be, timeout=datetime.timedelta(seconds=timeout_s), **kw)
        h = CommHandle(dist.get_rank(), dist.get_world_size(), None, True)
        h.timeout_s = timeout_s
        return h

    def subgroup(self, ranks: List[int]) -> "CommHandle":
        import torch.distributed as dist
        self._need()
        g = dist.new_group(ranks, timeout=datetime.timedelta(seconds=self.timeout_s))
        return CommHandle(ranks.index(self.rank) if self.rank in ranks else -1, len(ranks), g, True)

    def _need(self):
        if not self._init:
            raise CommError("communication handle is not initialised")

    def set_timeout(self, seconds: float):
        self.timeout_s = float(seconds)

    # ---- collectives ----------------------------------------------------------------------------
    def all_reduce(self, t: torch.Tensor, op: str = "sum", async_op: bool = False):
        import torch.distributed as dist
        self._need()
        ops = {"sum": dist.ReduceOp.SUM, "max": dist.ReduceOp.MAX, "min": dist.ReduceOp.MIN}
        return dist.all_reduce(t, op=ops[op], group=self.group, async_op=async_op)

    def reduce_scatter(self, out: torch.Tensor, inp: torch.Tensor, async_op: bool = False):
        import torch.distributed as dist
        self._need()
        if dist.get_backend(self.group) == "gloo":  # gloo has no reduce_scatter: all-reduce then slice
            tmp = inp.clone()
            dist.all_reduce(tmp, group=self.group)
            out.copy_(tmp.reshape(self.world_size, -1)[self.rank].reshape(out.shape))
            return None
        return dist.reduce_scatter_tensor(out, inp, group=self.group, async_op=async_op)

    def all_gather(self, out: torch.Tensor, inp: torch.Tensor, async_op: bool = False):
        import torch.distributed as dist
        self._need()
        return dist.all_gather_into_tensor(out, inp, group=self.group, async_op=async_op)

    def broadcast(self, t: torch.Tensor, src: int = 0, async_op: bool = False):
        import torch.distributed as dist
        self._need()
        return dist.broadcast(t, src=src, group=self.group, async_op=async_op)

    def all_to_all(self, out: torch.Tensor, inp: torch.Tensor, out_splits=None, in_splits=None):
        import torch.distributed as dist
        self._need()
        if dist.get_backend(self.group) == "gloo":
            outs = list(out.split(out_splits or out.shape[0] // self.world_size))
            ins = list(inp.split(in_splits or inp.shape[0] // self.world_size))
            return dist.all_to_all(outs, ins, group=self.group)
        return dist.all_to_all_single(out, inp, out_splits, in_splits, group=self.group)

    def send(self, t: torch.Tensor, dst: int, async_op: bool = False):
        import torch.distributed as dist
        self._need()
        return dist.isend(t, dst, group=self.group) if async_op else dist.send(t, dst, group=self.group)

    def recv(self, t: torch.Tensor, src: int, async_op: bool = False):
        import torch.distributed as dist
        self._need()
        return dist.irecv(t, src, group=self.group) if async_op else dist.recv(t, src, group=self.group)

    def all_reduce_counts(self, counts: torch.Tensor):
        """Integer counters (EPLB statistics) are reduced as int64, not cast to f32 as the reference does."""
        self._need()
        c = counts.to(torch.int64)
        self.all_reduce(c)
        return c

    def barrier(self):
        import torch.distributed as dist
        self._need()
        dist.barrier(group=self.group)

    def destroy(self):
        """Idempotent: barrier, then drop the process group (only when this handle owns the world group)."""
        import torch.distributed as dist
        if not self._init:
            return
        try:
            self.barrier()
        finally:
            self._init = False
            if self.group is None and dist.is_initialized():
                dist.destroy_process_group()
