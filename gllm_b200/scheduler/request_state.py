"""Per-request state table that kernels can read: one fixed-size record per slot, mirrored host <-> device.

Reference parity: src/scheduler/request_state.rs:18-490 (phase, exit flags, bus ports, CUDA upload). The host
copy is a numpy structured array in pinned memory; ``upload`` issues a single async copy.
"""
from __future__ import annotations

import enum

import numpy as np
import torch

REQUEST_STATE_DTYPE = np.dtype([
    ("request_id", "<u8"), ("phase", "u1"), ("exit_flags", "u1"), ("bus_ports", "<u2"), ("position", "<u4"),
    ("generated", "<u4"), ("max_tokens", "<u4"), ("eos_token", "<i4"), ("exit_layer", "<i2"), ("_pad", "V2"),
])
assert REQUEST_STATE_DTYPE.itemsize == 32


class Phase(enum.IntEnum):
    IDLE = 0
    PREFILL = 1
    DECODE = 2
    FINISHED = 3


class ExitFlag(enum.IntFlag):
    EOS = 1
    LENGTH = 2
    VETO = 4
    EARLY_EXIT = 8
    ABORT = 16


class RequestStateTable:
    def __init__(self, slots: int, device=None):
        self.slots = slots
        self.device = torch.device(device) if device is not None else None
        pin = self.device is not None and self.device.type == "cuda"
        self._host = torch.zeros(slots * REQUEST_STATE_DTYPE.itemsize, dtype=torch.uint8, pin_memory=pin)
        self.rec = self._host.numpy().view(REQUEST_STATE_DTYPE)
        self.dev = torch.zeros_like(self._host, device=self.device) if pin else None

    def assign(self, slot: int, request_id: int, max_tokens: int, eos_token: int = -1):
        r = self.rec[slot]
        r["request_id"], r["phase"], r["exit_flags"], r["position"], r["generated"] = request_id, Phase.PREFILL, 0, 0, 0
        r["max_tokens"], r["eos_token"], r["exit_layer"] = max_tokens, eos_token, -1

    def advance(self, slot: int, token: int):
        r = self.rec[slot]
        r["phase"] = Phase.DECODE
        r["generated"] += 1
        r["position"] += 1
        if token == r["eos_token"]:
            r["exit_flags"] |= ExitFlag.EOS
        if r["generated"] >= r["max_tokens"]:
            r["exit_flags"] |= ExitFlag.LENGTH
        if r["exit_flags"]:
            r["phase"] = Phase.FINISHED
        return int(r["exit_flags"])

    def advance_many(self, slots, tokens):
        """``advance`` for many slots at once (one decode step): numpy field arithmetic, no per-token Python work."""
        if len(slots) == 0:
            return
        r = self.rec
        slots = np.asarray(slots)
        tokens = np.asarray(tokens)
        r["generated"][slots] += 1
        r["position"][slots] += 1
        flags = r["exit_flags"][slots]
        flags = flags | np.where(tokens == r["eos_token"][slots], int(ExitFlag.EOS), 0).astype(np.uint8)
        flags = flags | np.where(r["generated"][slots] >= r["max_tokens"][slots], int(ExitFlag.LENGTH), 0).astype(np.uint8)
        r["exit_flags"][slots] = flags
        r["phase"][slots] = np.where(flags != 0, int(Phase.FINISHED), int(Phase.DECODE)).astype(np.uint8)

    def set_flag(self, slot: int, flag: ExitFlag):
        self.rec[slot]["exit_flags"] |= int(flag)
        self.rec[slot]["phase"] = Phase.FINISHED

    def open_port(self, slot: int, port: int):
        self.rec[slot]["bus_ports"] |= (1 << port)

    def release(self, slot: int):
        self.rec[slot] = np.zeros((), dtype=REQUEST_STATE_DTYPE)

    def upload(self):
        if self.dev is not None:
            self.dev.copy_(self._host, non_blocking=True)
        return self.dev
