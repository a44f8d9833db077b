"""Flat batch descriptor: one contiguous buffer with a 96-byte header and a 64-byte record per sequence, the
form in which a step's metadata crosses to the device in ONE pinned copy.

Reference parity: ``BatchContext`` 96 B header + 64 B/seq metadata (src/engine/batch_context.rs:21-167; v2
extension src/engine/mega_kernel_gpu.rs:27-106) and ``BatchExecutor`` flat sampling params
``[temp, top_k, top_p, eos] x N`` (src/engine/batch_executor.rs:18-579).
"""
from __future__ import annotations

import numpy as np
import torch

HEADER_DTYPE = np.dtype([
    ("magic", "<u4"), ("version", "<u4"), ("num_seqs", "<u4"), ("num_tokens", "<u4"), ("num_decode", "<u4"),
    ("num_prefill", "<u4"), ("max_q_len", "<u4"), ("max_ctx_len", "<u4"), ("page_size", "<u4"), ("max_blocks", "<u4"),
    ("step", "<u8"), ("seed", "<u8"), ("flags", "<u4"), ("_pad", "V36"),
])
SEQ_DTYPE = np.dtype([
    ("request_id", "<u8"), ("q_start", "<u4"), ("q_len", "<u4"), ("ctx_len", "<u4"), ("slot", "<i4"),
    ("temperature", "<f4"), ("top_k", "<i4"), ("top_p", "<f4"), ("eos", "<i4"), ("generated", "<u4"), ("max_tokens", "<u4"),
    ("block_table_off", "<u4"), ("flags", "<u4"), ("_pad", "V8"),
])
assert HEADER_DTYPE.itemsize == 96 and SEQ_DTYPE.itemsize == 64
MAGIC = 0x474C4C4D  # "GLLM"


class BatchContext:
    def __init__(self, max_seqs: int, pinned: bool = False):
        self.max_seqs = max_seqs
        self.buf = torch.zeros(96 + 64 * max_seqs, dtype=torch.uint8, pin_memory=pinned)
        raw = self.buf.numpy()
        self.header = raw[:96].view(HEADER_DTYPE)
        self.seqs = raw[96:].view(SEQ_DTYPE)
        self.header["magic"], self.header["version"] = MAGIC, 2

    def fill(self, seqs, *, step: int, seed: int, page_size: int = 16, max_blocks: int = 0):
        """``seqs``: iterable of dicts with request_id, q_len, ctx_len, slot, temperature, top_k, top_p, eos,
        generated, max_tokens."""
        seqs = list(seqs)
        if len(seqs) > self.max_seqs:
            raise ValueError("batch larger than the descriptor")
        h = self.header
        q = 0
        for i, s in enumerate(seqs):
            r = self.seqs[i]
            for k in ("request_id", "q_len", "ctx_len", "slot", "temperature", "top_k", "top_p", "eos", "generated", "max_tokens"):
                r[k] = s.get(k, 0)
            r["q_start"], r["block_table_off"] = q, i * max_blocks
            q += int(s["q_len"])
        h["num_seqs"], h["num_tokens"] = len(seqs), q
        h["num_decode"] = sum(1 for s in seqs if s["q_len"] == 1)
        h["num_prefill"] = len(seqs) - int(h["num_decode"][0])
        h["max_q_len"] = max((s["q_len"] for s in seqs), default=0)
        h["max_ctx_len"] = max((s["ctx_len"] for s in seqs), default=0)
        h["page_size"], h["max_blocks"], h["step"], h["seed"] = page_size, max_blocks, step, seed
        return self

    def sampling_params(self) -> torch.Tensor:
        """[N, 4] float32: temperature, top_k, top_p, eos."""
        n = int(self.header["num_seqs"][0])
        s = self.seqs[:n]
        return torch.from_numpy(np.stack([s["temperature"], s["top_k"].astype(np.float32), s["top_p"],
                                          s["eos"].astype(np.float32)], 1).astype(np.float32))

    def nbytes(self) -> int:
        return 96 + 64 * int(self.header["num_seqs"][0])

    def upload(self, device) -> torch.Tensor:
        return self.buf[: self.nbytes()].to(device, non_blocking=True)
