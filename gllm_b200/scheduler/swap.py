"""Three-tier swap: HBM <-> pinned host <-> NVMe file, with background eviction / swap-in workers, a migration
actor that executes DMA commands on a side stream, CRC16 integrity and page compression.

Reference parity: coordinator + workers + ``PageMigrationActor`` (commands EvictToDram / PromoteToHbm /
EvictToNvme / PromoteToDram) + ``DmaBackend`` implementations + O_DIRECT swap file + CRC16 + codecs
(src/scheduler/three_tier_swap.rs, eviction_worker.rs, swap_in_worker.rs, migration_actor.rs,
dma_helpers.rs:21-630, nvme_swap.rs). Policy numbers (trigger at HBM > 90 % / DRAM > 80 %; HBM->DRAM when
importance < 100 and age > 50 ticks; DRAM->NVMe when age > 500 ticks; NVMe promoted in two hops):
src/scheduler/eviction_worker.rs:1-40,117-160, src/scheduler/swap_in_worker.rs:1-60.

B200 mapping: the DMA backend issues one ``cudaMemcpyAsync`` per page (through ``Tensor.copy_(non_blocking)``)
between the device pool and a pinned host pool on a dedicated stream; the CPU backend is a memcpy. LZ4 / zstd
are not in this image: ``zlib`` stands in for both byte codecs, and the bit-pack RLE codec is implemented here.
"""
from __future__ import annotations

import enum
import os
import queue
import threading
import zlib
from dataclasses import dataclass
from typing import Callable, Dict, List, Optional, Tuple

import numpy as np
import torch

from ..kv_cache.header import CompressionCodec, StorageTier


# ------------------------------------------------------------------------------------------------
# integrity + codecs
# ------------------------------------------------------------------------------------------------
def crc16_ccitt(data: bytes, crc: int = 0xFFFF) -> int:
    table = _CRC_TABLE
    for b in data:
        crc = ((crc << 8) & 0xFFFF) ^ table[((crc >> 8) ^ b) & 0xFF]
    return crc


def _make_crc_table():
    t = []
    for i in range(256):
        c = i << 8
        for _ in range(8):
            c = ((c << 1) ^ 0x1021) & 0xFFFF if c & 0x8000 else (c << 1) & 0xFFFF
        t.append(c)
    return t


_CRC_TABLE = _make_crc_table()


def rle_bitpack_encode(data: bytes) -> bytes:
    """Byte-level run-length code: (count, value) pairs, count <= 255. Good on zero-heavy quantised pages."""
    a = np.frombuffer(data, dtype=np.uint8)
    if a.size == 0:
        return b""
    change = np.flatnonzero(np.diff(a)) + 1
    starts = np.concatenate([[0], change])
    lens = np.diff(np.concatenate([starts, [a.size]]))
    out = bytearray()
    for s, n in zip(starts.tolist(), lens.tolist()):
        v = int(a[s])
        while n > 0:
            c = min(n, 255)
            out += bytes((c, v))
            n -= c
    return bytes(out)


def rle_bitpack_decode(data: bytes) -> bytes:
    a = np.frombuffer(data, dtype=np.uint8).reshape(-1, 2)
    return np.repeat(a[:, 1], a[:, 0]).tobytes()


def compress(data: bytes, codec: CompressionCodec) -> bytes:
    if codec == CompressionCodec.NONE:
        return data
    if codec == CompressionCodec.BITPACK_RLE:
        return rle_bitpack_encode(data)
    level = 1 if codec == CompressionCodec.LZ4 else 6
    return zlib.compress(data, level)


def decompress(data: bytes, codec: CompressionCodec) -> bytes:
    if codec == CompressionCodec.NONE:
        return data
    if codec == CompressionCodec.BITPACK_RLE:
        return rle_bitpack_decode(data)
    return zlib.decompress(data)


# ------------------------------------------------------------------------------------------------
# DMA backends
# ------------------------------------------------------------------------------------------------
class LayeredPool:
    """The serving engine's KV cache: one device tensor [pages, ...] per layer. A "page" of this pool is the same
    page index in every layer, and its host image is [layers, ...]. Indexing and ``copy_`` are what the DMA
    backends use, so the pool stands in for a single stacked tensor without the cache having to be one allocation."""

    class _Page:
        def __init__(self, layers, page):
            self.layers, self.page = layers, page

        def copy_(self, host_page, non_blocking=False):          # host image -> device page
            for l, t in enumerate(self.layers):
                t[self.page].copy_(host_page[l], non_blocking=non_blocking)

    def __init__(self, layers: List[torch.Tensor]):
        self.layers = list(layers)
        t = self.layers[0]
        self.shape = (t.shape[0], len(self.layers)) + tuple(t.shape[1:])
        self.dtype, self.device, self.is_cuda = t.dtype, t.device, t.is_cuda

    def __getitem__(self, page: int):
        return LayeredPool._Page(self.layers, page)


def _copy_page_to_host(host_page: torch.Tensor, dev_page, non_blocking=False):
    if isinstance(dev_page, LayeredPool._Page):
        for l, t in enumerate(dev_page.layers):
            host_page[l].copy_(t[dev_page.page], non_blocking=non_blocking)
    else:
        host_page.copy_(dev_page, non_blocking=non_blocking)


class DmaBackend:
    def d2h(self, dev_pool: torch.Tensor, page: int, host_pool: torch.Tensor, slot: int):
        raise NotImplementedError

    def h2d(self, host_pool: torch.Tensor, slot: int, dev_pool: torch.Tensor, page: int):
        raise NotImplementedError

    def synchronize(self):
        pass


class MemcpyDma(DmaBackend):
    def d2h(self, dev_pool, page, host_pool, slot):
        _copy_page_to_host(host_pool[slot], dev_pool[page])

    def h2d(self, host_pool, slot, dev_pool, page):
        dev_pool[page].copy_(host_pool[slot])


class CudaStreamDma(DmaBackend):
    """One async copy per page on a dedicated stream; the compute stream never waits unless it asks to."""

    def __init__(self, device):
        self.stream = torch.cuda.Stream(device=device)

    def d2h(self, dev_pool, page, host_pool, slot):
        self.stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(self.stream):
            _copy_page_to_host(host_pool[slot], dev_pool[page], non_blocking=True)

    def h2d(self, host_pool, slot, dev_pool, page):
        with torch.cuda.stream(self.stream):
            dev_pool[page].copy_(host_pool[slot], non_blocking=True)

    def synchronize(self):
        self.stream.synchronize()


# ------------------------------------------------------------------------------------------------
# NVMe swap file
# ------------------------------------------------------------------------------------------------
class NvmeSwapFile:
    """Fixed-size slots in one file. Each record: 8-byte header (codec, crc16, length) + payload."""

    def __init__(self, path: str, slot_bytes: int, slots: int):
        self.path, self.slot_bytes, self.slots = path, slot_bytes + 8, slots
        self.fd = os.open(path, os.O_RDWR | os.O_CREAT, 0o600)
        os.ftruncate(self.fd, self.slot_bytes * slots)
        self.free = list(range(slots - 1, -1, -1))

    def write(self, data: bytes, codec: CompressionCodec) -> int:
        payload = compress(data, codec)
        if len(payload) > self.slot_bytes - 8:
            payload, codec = data, CompressionCodec.NONE
        slot = self.free.pop()
        hdr = bytes((int(codec), 0)) + crc16_ccitt(data).to_bytes(2, "little") + len(payload).to_bytes(4, "little")
        os.pwrite(self.fd, hdr + payload, slot * self.slot_bytes)
        return slot

    def read(self, slot: int, release: bool = True) -> bytes:
        hdr = os.pread(self.fd, 8, slot * self.slot_bytes)
        codec, crc, n = CompressionCodec(hdr[0]), int.from_bytes(hdr[2:4], "little"), int.from_bytes(hdr[4:8], "little")
        data = decompress(os.pread(self.fd, n, slot * self.slot_bytes + 8), codec)
        if crc16_ccitt(data) != crc:
            raise IOError(f"swap slot {slot}: CRC mismatch")
        if release:
            self.free.append(slot)
        return data

    def close(self):
        os.close(self.fd)
        try:
            os.unlink(self.path)
        except OSError:
            pass


# ------------------------------------------------------------------------------------------------
# migration actor + workers
# ------------------------------------------------------------------------------------------------
class DmaCommand(enum.Enum):
    EVICT_TO_DRAM = 0
    PROMOTE_TO_HBM = 1
    EVICT_TO_NVME = 2
    PROMOTE_TO_DRAM = 3


@dataclass
class PageRecord:
    tier: StorageTier
    location: int          # device page, host slot or file slot
    importance: int = 128
    age: int = 0
    codec: CompressionCodec = CompressionCodec.NONE


@dataclass
class SwapPolicy:
    hbm_trigger: float = 0.90
    dram_trigger: float = 0.80
    hbm_importance_below: int = 100
    hbm_age_above: int = 50
    dram_age_above: int = 500
    dram_codec: CompressionCodec = CompressionCodec.LZ4
    nvme_codec: CompressionCodec = CompressionCodec.ZSTD_DICT


class ThreeTierSwap:
    """Coordinator. ``dev_pool`` [pages, ...] is the device KV pool (one stacked tensor, or a ``LayeredPool`` over the
    per-layer caches of the serving engine), ``host_slots`` pinned host pages of one page's shape."""

    def __init__(self, dev_pool, host_slots: int, swap_path: Optional[str] = None, nvme_slots: int = 0,
                 policy: SwapPolicy = SwapPolicy(), dma: Optional[DmaBackend] = None):
        self.dev_pool = dev_pool
        pin = dev_pool.is_cuda
        hdt = torch.uint8 if dev_pool.dtype == torch.float8_e4m3fn else dev_pool.dtype
        self.host_pool = torch.zeros((host_slots,) + tuple(dev_pool.shape[1:]), dtype=hdt, pin_memory=pin)
        self.host_free = list(range(host_slots - 1, -1, -1))
        self.dev_free: List[int] = []
        self.policy = policy
        self.dma = dma or (CudaStreamDma(dev_pool.device) if dev_pool.is_cuda else MemcpyDma())
        self.page_bytes = self.host_pool[0].numel() * self.host_pool.element_size() if host_slots else 0
        self.nvme = NvmeSwapFile(swap_path, self.page_bytes, nvme_slots) if swap_path and nvme_slots else None
        self.records: Dict[int, PageRecord] = {}       # logical page key -> where it lives
        self.lock = threading.Lock()
        self.stats = {"evict_dram": 0, "evict_nvme": 0, "promote_hbm": 0, "promote_dram": 0}

    def register(self, key: int, dev_page: int, importance: int = 128):
        self.records[key] = PageRecord(StorageTier.HBM, dev_page, importance)

    def execute(self, cmd: DmaCommand, key: int, dev_page: Optional[int] = None):
        with self.lock:
            r = self.records[key]
            if cmd == DmaCommand.EVICT_TO_DRAM:
                assert r.tier == StorageTier.HBM
                slot = self.host_free.pop()
                self.dma.d2h(self.dev_pool, r.location, self.host_pool, slot)
                self.dma.synchronize()
                self.dev_free.append(r.location)
                r.tier, r.location, r.age = StorageTier.DRAM, slot, 0
                self.stats["evict_dram"] += 1
            elif cmd == DmaCommand.PROMOTE_TO_HBM:
                if r.tier == StorageTier.NVME:      # two hops
                    self._promote_to_dram(r)
                assert r.tier == StorageTier.DRAM
                page = dev_page if dev_page is not None else self.dev_free.pop()
                self.dma.h2d(self.host_pool, r.location, self.dev_pool, page)
                self.dma.synchronize()
                self.host_free.append(r.location)
                r.tier, r.location, r.age = StorageTier.HBM, page, 0
                self.stats["promote_hbm"] += 1
            elif cmd == DmaCommand.EVICT_TO_NVME:
                assert r.tier == StorageTier.DRAM and self.nvme is not None
                raw = self.host_pool[r.location].contiguous().view(torch.uint8).numpy().tobytes()
                slot = self.nvme.write(raw, self.policy.nvme_codec)
                self.host_free.append(r.location)
                r.tier, r.location, r.age, r.codec = StorageTier.NVME, slot, 0, self.policy.nvme_codec
                self.stats["evict_nvme"] += 1
            elif cmd == DmaCommand.PROMOTE_TO_DRAM:
                self._promote_to_dram(r)
        return self.records[key]

    def _promote_to_dram(self, r: PageRecord):
        assert r.tier == StorageTier.NVME
        data = self.nvme.read(r.location)
        slot = self.host_free.pop()
        self.host_pool[slot].view(torch.uint8).reshape(-1).copy_(torch.frombuffer(bytearray(data), dtype=torch.uint8))
        r.tier, r.location, r.age = StorageTier.DRAM, slot, 0
        self.stats["promote_dram"] += 1

    # ---- policy passes (what the background workers run) --------------------------------------------
    def tick(self):
        for r in self.records.values():
            r.age += 1

    def eviction_pass(self, hbm_used_ratio: float, dram_used_ratio: Optional[float] = None) -> List[Tuple[DmaCommand, int]]:
        p = self.policy
        cmds = []
        if hbm_used_ratio > p.hbm_trigger:
            for key, r in sorted(self.records.items(), key=lambda kv: kv[1].importance):
                if r.tier == StorageTier.HBM and r.importance < p.hbm_importance_below and r.age > p.hbm_age_above \
                        and len(self.host_free) > len(cmds):
                    cmds.append((DmaCommand.EVICT_TO_DRAM, key))
        if dram_used_ratio is None:
            dram_used_ratio = 1.0 - len(self.host_free) / max(self.host_pool.shape[0], 1)
        if self.nvme is not None and dram_used_ratio > p.dram_trigger:
            for key, r in self.records.items():
                if r.tier == StorageTier.DRAM and r.age > p.dram_age_above:
                    cmds.append((DmaCommand.EVICT_TO_NVME, key))
        for c, k in cmds:
            self.execute(c, k)
        return cmds

    @staticmethod
    def swap_in_urgency(score_rebound: float, prefetch_confidence: float, tier: StorageTier) -> float:
        return score_rebound + prefetch_confidence + 1.0 / (1 + int(tier))

    def close(self):
        if self.nvme:
            self.nvme.close()


class BackgroundWorker(threading.Thread):
    """Runs ``fn`` on items from a queue until stopped (eviction worker / swap-in worker)."""

    def __init__(self, fn: Callable, name: str):
        super().__init__(name=name, daemon=True)
        self.fn, self.q, self.done = fn, queue.Queue(), queue.Queue()
        self._halt = threading.Event()

    def submit(self, item):
        self.q.put(item)

    def run(self):
        while not self._halt.is_set():
            try:
                item = self.q.get(timeout=0.05)
            except queue.Empty:
                continue
            try:
                self.done.put((item, self.fn(item), None))
            except Exception as exc:   # reported to the submitter, the worker keeps running
                self.done.put((item, None, exc))

    def stop(self):
        self._halt.set()
        self.join(timeout=2)
