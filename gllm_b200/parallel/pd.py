"""Prefill / decode disaggregation, KV page transfer between roles, KV distribution modes, and the SAGUARO
draft / verify hand-off.

Reference parity: ``PdRoleDecision{Collocated, PrefillOnly, DecodeOnly}`` and step gating
(src/engine/coordinator/dispatch.rs:34-60, executor_step.rs:121-250), ``kv_transfer / send_pages / recv_pages``
(src/engine/coordinator/kv.rs:395-569; synchronous underneath in the reference — here the transfer is issued on
a side stream and returns a handle), ``KvDistMode`` behaviours (coordinator/kv.rs:52-156), SAGUARO token
hand-off via ``send_bytes / recv_bytes`` (src/speculative/saguaro.rs:35-490).
"""
from __future__ import annotations

import time
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import torch

from .config import KvDistMode, PdRole


def resolve_pd_role(role: PdRole, has_prefill_work: bool, has_decode_work: bool) -> Dict[str, bool]:
    """Which phases a rank runs this step."""
    if role == PdRole.PREFILL_ONLY:
        return {"prefill": has_prefill_work, "decode": False, "ship_kv": has_prefill_work}
    if role == PdRole.DECODE_ONLY:
        return {"prefill": False, "decode": has_decode_work, "ship_kv": False}
    return {"prefill": has_prefill_work, "decode": has_decode_work, "ship_kv": False}


@dataclass
class KvTransferResult:
    pages: int
    bytes: int
    latency_ms: float


class KvPageTransport:
    """Moves whole KV pages (all layers of a page id) between two ranks."""

    def __init__(self, comm, kv_caches: List[torch.Tensor]):
        self.comm, self.kv = comm, kv_caches
        dev = kv_caches[0].device
        self.stream = torch.cuda.Stream(device=dev) if dev.type == "cuda" else None

    def _gather(self, pages: Sequence[int]) -> torch.Tensor:
        idx = torch.as_tensor(list(pages), dtype=torch.long, device=self.kv[0].device)
        return torch.stack([c.index_select(0, idx) for c in self.kv]).contiguous()   # [L, n, 2, Hkv, 16, D]

    def send_pages(self, pages: Sequence[int], dst: int) -> KvTransferResult:
        t0 = time.perf_counter()
        buf = self._gather(pages)
        self.comm.send(buf, dst)
        return KvTransferResult(len(pages), buf.numel() * buf.element_size(), (time.perf_counter() - t0) * 1e3)

    def recv_pages(self, pages: Sequence[int], src: int) -> KvTransferResult:
        t0 = time.perf_counter()
        shape = (len(self.kv), len(pages)) + tuple(self.kv[0].shape[1:])
        buf = torch.empty(shape, dtype=self.kv[0].dtype, device=self.kv[0].device)
        self.comm.recv(buf, src)
        idx = torch.as_tensor(list(pages), dtype=torch.long, device=self.kv[0].device)
        for l, c in enumerate(self.kv):
            c.index_copy_(0, idx, buf[l])
        return KvTransferResult(len(pages), buf.numel() * buf.element_size(), (time.perf_counter() - t0) * 1e3)


def kv_dist_plan(mode: KvDistMode, rank: int, world: int, n_kv_heads: int) -> Dict[str, object]:
    """What a rank stores under each KV distribution mode."""
    if mode == KvDistMode.LOCAL:
        return {"store_heads": list(range(n_kv_heads)), "fetch_on_miss": False, "mirror_to": []}
    if mode == KvDistMode.ON_DEMAND:
        return {"store_heads": list(range(n_kv_heads)), "fetch_on_miss": True, "mirror_to": []}
    if mode == KvDistMode.MIRROR:
        return {"store_heads": list(range(n_kv_heads)), "fetch_on_miss": False,
                "mirror_to": [r for r in range(world) if r != rank]}
    if mode == KvDistMode.PARTIAL_HEAD_MIRROR:
        per = max(1, n_kv_heads // world)
        own = list(range(rank * per, min(n_kv_heads, (rank + 1) * per)))
        return {"store_heads": own, "fetch_on_miss": True, "mirror_to": [(rank + 1) % world]}
    return {"store_heads": list(range(n_kv_heads)), "fetch_on_miss": True, "mirror_to": [], "tiered": True}


class KvDistributor:
    """The KV distribution modes over a set of serving engines reachable as objects: the engines of one process (one
    per GPU of a node, each e.g. behind its own ``ServingLoop``); page tensors move device to device with ``.to()``.
    Engines of different processes hand pages over with the ``engine.pd`` links instead.

    LOCAL: nothing moves. MIRROR: after a request finishes, the full pages of its conversation are copied into every
    peer's prefix cache, so the next turn may land anywhere. ON_DEMAND (and TIERED / PARTIAL_HEAD_MIRROR for the part
    that fetches): before a request is admitted on a rank whose cache misses its prefix, the longest cached prefix
    any peer holds is fetched. Pages arrive as cached prefix pages (``LLMEngine.import_prefix_pages``); the admission
    then computes only what is missing. Reference: KvDistMode behaviours (src/engine/coordinator/kv.rs:52-156, 395-569)."""

    def __init__(self, engines: Dict[int, object], mode: KvDistMode):
        self.engines, self.mode = dict(engines), mode
        self.stats = {"mirrored_pages": 0, "fetched_pages": 0, "fetches": 0}

    def after_finish(self, rank: int, tokens: Sequence[int]) -> int:
        """Call with the conversation's tokens (prompt + generated) once a request has finished on ``rank``."""
        plan = kv_dist_plan(self.mode, rank, len(self.engines), 1)
        if not plan["mirror_to"]:
            return 0
        n, pages = self.engines[rank].export_prefix_pages(list(tokens))
        moved = 0
        for peer in plan["mirror_to"]:
            if n and peer in self.engines:
                moved += self.engines[peer].import_prefix_pages(list(tokens), pages)
        self.stats["mirrored_pages"] += moved
        return moved

    def before_admit(self, rank: int, tokens: Sequence[int]) -> int:
        """Call before ``add_request`` on ``rank``: fetches the longest prefix a peer has cached and this rank lacks."""
        plan = kv_dist_plan(self.mode, rank, len(self.engines), 1)
        if not plan["fetch_on_miss"]:
            return 0
        toks = list(tokens)
        mine = len(self.engines[rank].batcher.lookup_prefix_pages([int(t) for t in toks[:len(toks) // 16 * 16]]))
        best, best_n = None, mine
        for peer, eng in self.engines.items():
            if peer == rank:
                continue
            n = len(eng.batcher.lookup_prefix_pages([int(t) for t in toks[:len(toks) // 16 * 16]]))
            if n > best_n:
                best, best_n = peer, n
        if best is None:
            return 0
        n, pages = self.engines[best].export_prefix_pages(toks)
        got = self.engines[rank].import_prefix_pages(toks, pages)
        self.stats["fetches"] += 1
        self.stats["fetched_pages"] += got
        return got


# ------------------------------------------------------------------------------------------------
# SAGUARO: draft rank proposes, verify rank checks (tens of bytes per round)
# ------------------------------------------------------------------------------------------------
class SaguaroLink:
    def __init__(self, comm, draft_rank: int, verify_rank: int, max_draft: int = 16):
        self.comm, self.draft_rank, self.verify_rank, self.max_draft = comm, draft_rank, verify_rank, max_draft

    def send_draft(self, tokens: Sequence[int]):
        buf = torch.full((self.max_draft + 1,), -1, dtype=torch.int32)
        buf[0] = len(tokens)
        buf[1:1 + len(tokens)] = torch.as_tensor(list(tokens), dtype=torch.int32)
        self.comm.send(buf, self.verify_rank)

    def recv_draft(self) -> List[int]:
        buf = torch.empty(self.max_draft + 1, dtype=torch.int32)
        self.comm.recv(buf, self.draft_rank)
        return buf[1:1 + int(buf[0])].tolist()

    def send_tokens(self, tokens: Sequence[int], dst: int, cap="draft", length_field=None):
        """A variable-length token message: one int32 header [length or a negative control code, capacity], then the
        body. ``cap=None`` sizes the body to the message (prompts); the default body has ``max_draft + 1`` slots."""
        n = len(tokens)
        size = n if cap is None else self.max_draft + 1
        if n > size:
            raise ValueError(f"{n} tokens do not fit a message of {size}")
        self.comm.send(torch.tensor([n if length_field is None else length_field, size], dtype=torch.int32), dst)
        if size:
            body = torch.full((size,), -1, dtype=torch.int32)
            body[:n] = torch.as_tensor(list(tokens), dtype=torch.int32)
            self.comm.send(body, dst)

    def recv_tokens(self, src: int, cap="draft"):
        """(tokens, length field) of a ``send_tokens`` message."""
        head = torch.empty(2, dtype=torch.int32)
        self.comm.recv(head, src)
        n, size = int(head[0]), int(head[1])
        body = torch.empty(size, dtype=torch.int32)
        if size:
            self.comm.recv(body, src)
        return body[:max(n, 0)].tolist(), n

    def send_verdict(self, accepted: int, correction: int):
        self.comm.send(torch.tensor([accepted, correction], dtype=torch.int32), self.draft_rank)

    def recv_verdict(self):
        buf = torch.empty(2, dtype=torch.int32)
        self.comm.recv(buf, self.verify_rank)
        return int(buf[0]), int(buf[1])
