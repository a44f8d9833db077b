"""Pipeline-parallel inference: every rank holds the decoder layers of one stage (and its slice of the KV
cache); hidden states travel stage to stage, sampled tokens travel from the last stage back to the first.

Micro-batches keep the stages busy: in each step stage s works on micro-batch j while stage s+1 works on j-1
(forward-only GPipe order). Sends are asynchronous (NCCL p2p on GPUs, gloo on CPU), so a stage overlaps the
transfer of micro-batch j with the compute of j+1. With tensor parallelism inside a stage, rank (tp=i, stage s)
talks to rank (tp=i, stage s+1): activations are replicated inside a TP group, so no extra broadcast is needed.

Reference parity: ``ActivationTransport`` send / recv of ``micro_batch * hidden`` values between stages
(src/engine/pipeline/activation_xfer.rs:151-560), the micro-batch schedulers
(src/engine/pipeline/scheduler.rs:135-375) and the per-stage KV manager (:884-1080).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence

import torch

from ...engine.batch import ForwardBatch
from . import PipelineConfig, split_micro_batches

PAGE = 16


@dataclass
class _Micro:
    seq_ids: List[int]
    page0: List[int]            # first page of each sequence in this stage's pool
    lens: List[int]             # tokens currently in the KV cache per sequence


class PipelineStageRunner:
    def __init__(self, model, comm, stage: int, num_stages: int, prev_rank: Optional[int], next_rank: Optional[int],
                 first_rank: int, last_rank: int, max_seq_len: int = 512):
        self.model, self.comm, self.stage, self.num_stages = model, comm, stage, num_stages
        self.prev, self.next, self.first_rank, self.last_rank = prev_rank, next_rank, first_rank, last_rank
        self.pages_per_seq = (max_seq_len + PAGE - 1) // PAGE
        self.dev, self.dtype = model.device, model.dtype
        self.H = model.cfg.hidden_size
        self.kv = None
        self.stats = {"sent_bytes": 0, "recv_bytes": 0, "forwards": 0}

    @property
    def is_first(self):
        return self.stage == 0

    @property
    def is_last(self):
        return self.stage == self.num_stages - 1

    # ---- batches ------------------------------------------------------------------------------------
    def _block_tables(self, mb: _Micro):
        bt = torch.zeros((len(mb.seq_ids), self.pages_per_seq), dtype=torch.int32, device=self.dev)
        for i, p0 in enumerate(mb.page0):
            bt[i] = torch.arange(p0, p0 + self.pages_per_seq, dtype=torch.int32, device=self.dev)
        return bt

    def _prefill_batch(self, mb: _Micro, prompts: Sequence[Sequence[int]]) -> ForwardBatch:
        lens = [len(p) for p in prompts]
        starts = [0]
        for n in lens[:-1]:
            starts.append(starts[-1] + n)
        i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=self.dev)
        slots = torch.cat([mb.page0[i] * PAGE + torch.arange(n, dtype=torch.int32, device=self.dev) for i, n in enumerate(lens)])
        rows = torch.tensor([s + n - 1 for s, n in zip(starts, lens)], dtype=torch.int64, device=self.dev)
        return ForwardBatch(token_ids=i32([t for p in prompts for t in p]),
                            positions=torch.cat([torch.arange(n, dtype=torch.int32, device=self.dev) for n in lens]),
                            slot_mapping=slots, block_tables=self._block_tables(mb), ctx_lens=i32(lens), q_start=i32(starts),
                            q_len=i32(lens), max_q_len=max(lens), logits_rows=rows)

    def _decode_batch(self, mb: _Micro, tokens: torch.Tensor) -> ForwardBatch:
        i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=self.dev)
        pos = i32(mb.lens)
        slots = i32([p0 * PAGE + n for p0, n in zip(mb.page0, mb.lens)])
        return ForwardBatch(token_ids=tokens.to(torch.int32), positions=pos, slot_mapping=slots,
                            block_tables=self._block_tables(mb), ctx_lens=pos + 1, is_decode=True)

    # ---- transport ----------------------------------------------------------------------------------
    def _recv_hidden(self, T: int) -> torch.Tensor:
        buf = torch.empty((T, self.H), dtype=self.dtype, device=self.dev)
        self.comm.recv(buf, self.prev)
        self.stats["recv_bytes"] += buf.numel() * buf.element_size()
        return buf

    def _send_hidden(self, x: torch.Tensor, pending: list):
        x = x.contiguous().clone()           # the workspace row is reused by the next micro-batch
        pending.append((self.comm.send(x, self.next, async_op=True), x))
        self.stats["sent_bytes"] += x.numel() * x.element_size()

    def _tokens_to_first(self, tok: Optional[torch.Tensor], n: int) -> torch.Tensor:
        """Last stage -> first stage (and nobody else needs them)."""
        if self.num_stages == 1:
            return tok
        if self.is_last:
            self.comm.send(tok.to(torch.int32).contiguous(), self.first_rank)
            return tok
        if self.is_first:
            buf = torch.empty(n, dtype=torch.int32, device=self.dev)
            self.comm.recv(buf, self.last_rank)
            return buf
        return None

    # ---- one pipeline pass over all micro-batches ----------------------------------------------------------
    def _pass(self, micro: List[_Micro], make_batch, token_counts: List[int]) -> List[Optional[torch.Tensor]]:
        pending, outs = [], []
        for j, mb in enumerate(micro):
            batch = make_batch(j, mb)
            hidden_in = None if self.is_first else self._recv_hidden(token_counts[j])
            y = self.model.forward(batch, self.kv, hidden_in=hidden_in)
            self.stats["forwards"] += 1
            if self.is_last:
                V = self.model.cfg.vocab_size
                outs.append(y[:, :V].argmax(-1).to(torch.int32))
            else:
                self._send_hidden(y, pending)
                outs.append(None)
        for work, _keep in pending:
            if work is not None:
                work.wait()
        return outs

    def generate_greedy(self, prompts: Sequence[Sequence[int]], max_new_tokens: int, micro_batches: int = 2) -> Optional[List[List[int]]]:
        """All ranks call this with the same prompts. The first-stage rank returns the generated ids; the others
        return None."""
        n = len(prompts)
        splits = split_micro_batches(n, min(micro_batches, n))
        self.kv = self.model.alloc_kv_cache(n * self.pages_per_seq + 1)
        micro = []
        for start, size in splits:
            ids = list(range(start, start + size))
            micro.append(_Micro(ids, [i * self.pages_per_seq for i in ids], [0] * size))
        # prefill
        tok = self._pass(micro, lambda j, mb: self._prefill_batch(mb, [prompts[i] for i in mb.seq_ids]),
                         [sum(len(prompts[i]) for i in mb.seq_ids) for mb in micro])
        for mb in micro:
            mb.lens = [len(prompts[i]) for i in mb.seq_ids]
        out = [[] for _ in range(n)]
        cur = [self._tokens_to_first(tok[j], len(mb.seq_ids)) for j, mb in enumerate(micro)]
        for step in range(max_new_tokens):
            if self.is_first:
                for j, mb in enumerate(micro):
                    for i, sid in enumerate(mb.seq_ids):
                        out[sid].append(int(cur[j][i]))
            if step == max_new_tokens - 1:
                break

            def mk(j, mb):
                t = cur[j] if self.is_first else torch.zeros(len(mb.seq_ids), dtype=torch.int32, device=self.dev)
                return self._decode_batch(mb, t)
            tok = self._pass(micro, mk, [len(mb.seq_ids) for mb in micro])
            for mb in micro:
                mb.lens = [l + 1 for l in mb.lens]
            cur = [self._tokens_to_first(tok[j], len(mb.seq_ids)) for j, mb in enumerate(micro)]
        return out if self.is_first else None


def build_stage_runner(cfg, src, comm, *, pp: int, tp: int = 1, device="cpu", dtype=torch.float32, tp_ctx=None,
                       max_seq_len: int = 512, max_positions: int = 1024) -> PipelineStageRunner:
    """Rank layout: rank = stage * tp + tp_index (pipeline stages are the slow dimension, so a TP group sits on
    neighbouring GPUs)."""
    from ...models.decoder import DecoderModel
    rank = comm.rank
    stage, tpi = rank // tp, rank % tp
    layers = PipelineConfig(num_layers=cfg.num_layers, num_stages=pp).stage_ranges()[stage]
    model = DecoderModel(cfg, src, device=device, dtype=dtype, tp=tp_ctx, max_positions=max_positions, layers=layers)
    prev_rank = None if stage == 0 else (stage - 1) * tp + tpi
    next_rank = None if stage == pp - 1 else (stage + 1) * tp + tpi
    return PipelineStageRunner(model, comm, stage, pp, prev_rank, next_rank, first_rank=tpi, last_rank=(pp - 1) * tp + tpi,
                               max_seq_len=max_seq_len)
