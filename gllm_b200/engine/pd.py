"""Prefill / decode disaggregation as engine roles.

A ``prefill_only`` engine runs prompts through prefill, samples the first token (that is the request's TTFT), and hands
the request over: its prompt, sampling parameters and the KV pages its prompt filled. A ``decode_only`` engine imports
those pages into its own pool as cached prefix pages and admits the request; the admission then finds every full page
of the prompt in the prefix cache, so only the last partial page (fewer than 16 tokens) is computed again before
decoding starts. ``collocated`` engines do both, as before.

Reference parity: ``PdRoleDecision{Collocated, PrefillOnly, DecodeOnly}`` and the step gating around it
(src/engine/coordinator/dispatch.rs:34-60, src/engine/executor_step.rs:121-250: PrefillOnly ends a step with
``pd_transfer_kv_pages``, DecodeOnly begins one with ``pd_receive_kv_pages``), page transfer
(src/engine/coordinator/kv.rs:395-569). The link is an interface: in one process a queue, across ranks the
``KvPageTransport`` of ``parallel/pd.py`` (NCCL / gloo p2p) for the pages plus a small metadata message.
"""
from __future__ import annotations

import collections
import pickle
from dataclasses import dataclass, field
from typing import Deque, List, Optional

import torch


@dataclass
class PdHandoff:
    request_id: int
    prompt: List[int]
    first_token: int
    params: dict                       # max_tokens, temperature, top_k, top_p, eos_ids
    pages: Optional[torch.Tensor]      # [layers, n_full_pages, ...page shape] KV of the prompt's full pages
    page_tokens: int = 16


class InProcessPdLink:
    """Hand-offs between two engines of one process (tests, single-node set-ups with separate CUDA streams)."""

    nonblocking = True      # poll() returns at once: a decode_only engine drains it at the start of every step

    def __init__(self):
        self.q: Deque[PdHandoff] = collections.deque()

    def send(self, h: PdHandoff):
        self.q.append(h)

    def poll(self) -> List[PdHandoff]:
        out = list(self.q)
        self.q.clear()
        return out


class CommPdLink:
    """Hand-offs between two ranks over a ``parallel.comm.CommHandle`` (NCCL on GPUs, gloo on CPU): a fixed-size header,
    the pickled metadata, then the page tensor."""

    nonblocking = False     # recv() waits for the peer: the serving loop calls import_handoff(link.recv()) itself

    def __init__(self, comm, peer: int, device="cpu"):
        self.comm, self.peer, self.device = comm, peer, torch.device(device)

    def send(self, h: PdHandoff):
        meta = pickle.dumps((h.request_id, h.prompt, h.first_token, h.params, h.page_tokens,
                             None if h.pages is None else (tuple(h.pages.shape), str(h.pages.dtype))))
        hdr = torch.tensor([len(meta)], dtype=torch.int64, device=self.device)
        self.comm.send(hdr, self.peer)
        self.comm.send(torch.frombuffer(bytearray(meta), dtype=torch.uint8).to(self.device), self.peer)
        if h.pages is not None:
            self.comm.send(h.pages.contiguous(), self.peer)

    def recv(self) -> PdHandoff:
        hdr = torch.zeros(1, dtype=torch.int64, device=self.device)
        self.comm.recv(hdr, self.peer)
        buf = torch.zeros(int(hdr[0]), dtype=torch.uint8, device=self.device)
        self.comm.recv(buf, self.peer)
        rid, prompt, first, params, page_tokens, pinfo = pickle.loads(bytes(buf.cpu().numpy()))
        pages = None
        if pinfo is not None:
            shape, dt = pinfo
            pages = torch.empty(shape, dtype=getattr(torch, dt.split(".")[-1]), device=self.device)
            self.comm.recv(pages, self.peer)
        return PdHandoff(rid, prompt, first, params, pages, page_tokens)

    def poll(self) -> List[PdHandoff]:     # the caller knows how many to expect; one blocking receive per call
        return [self.recv()]
