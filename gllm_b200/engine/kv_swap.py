"""Swap tier of the serving engine: sequences preempted under memory pressure leave for pinned host memory (and,
when that fills up, for the NVMe file) instead of being recomputed, and come back when pages are free.

The C++ batcher decides WHEN (``PolicyConfig.preempt_swap``: its plans list ``swap_out`` / ``swap_in`` items), this
module decides WHO (``Hgal``: gang-aware eviction order over the running sequences, handed to the batcher as its
victim order) and moves the bytes (``ThreeTierSwap`` over a ``LayeredPool`` view of the per-layer KV caches: one page
of the pool is the same page index in every layer).

Reference parity: ``reclaim_memory`` / ``ensure_pages_resident`` / ``check_memory_pressure``
(src/engine/executor.rs:736-1050) on top of ``ThreeTierSwapCoordinator`` (src/scheduler/three_tier_swap.rs) with
``HGALScheduler::select_victims`` choosing whole sequence groups (src/scheduler/hgal.rs:111-156,306-331).
"""
from __future__ import annotations

import time
from typing import Dict, List, Optional

import torch

from ..kv_cache.header import StorageTier
from ..scheduler.hgal import Hgal, HgalConfig
from ..scheduler.swap import DmaCommand, LayeredPool, SwapPolicy, ThreeTierSwap
from ..scheduler.types import PayloadKind, UnifiedVirtualPage


class KvSwapManager:
    def __init__(self, kv_caches: List[torch.Tensor], host_pages: int, *, swap_path: Optional[str] = None,
                 nvme_pages: int = 0, hgal: Optional[HgalConfig] = None, device_pool_pages: int = 0):
        layers = [t.view(torch.uint8) if t.dtype == torch.float8_e4m3fn else t for t in kv_caches]
        # the 4-bit tier on the device itself (bf16 / fp32 caches in the [pages, 2, n_kv, 16, D] layout only)
        self.device_tier = None
        self.tier_policy = None        # callable(seq_id) -> PrecisionTier the sequence may wait in (None: KIVI4)
        # the packed tier keeps the sequence's attention-sink tokens (its first tokens) in 16 bit, as the TurboQuant
        # runtime of the KV cache does: the pages that hold them take the lossless host path
        from ..kv_cache.turboquant import TurboQuantConfig
        self.turboquant = TurboQuantConfig(enabled=device_pool_pages > 0)
        self.sink_pages = (self.turboquant.sink_tokens + 15) // 16 if self.turboquant.enabled else 0
        self.sink_keys: Dict[int, List[int]] = {}  # sequence packed on the device -> host keys of its lossless pages
        self.layout: Dict[int, list] = {}          # sequence packed on the device -> per logical page ("host", key) | ("pool", slot)
        self.page_tier = None                      # callable(page) -> PrecisionTier from the page headers (KV telemetry)
        self.packed: Dict[int, List[int]] = {}     # sequence packed on the device -> its pool slots, logical order
        if device_pool_pages > 0 and kv_caches[0].dim() == 5 and kv_caches[0].dtype != torch.float8_e4m3fn:
            from ..kv_cache.device_tier import Kivi4Pool
            self.device_tier = Kivi4Pool(kv_caches, device_pool_pages)
        self.swap = ThreeTierSwap(LayeredPool(layers), host_pages, swap_path=swap_path, nvme_slots=nvme_pages,
                                  policy=SwapPolicy())
        # victims must be allowed right away in a serving step: the warm-up window only protects pages from the
        # background eviction passes of the reference, not from the batcher's own out-of-memory handling
        self.hgal = Hgal(hgal or HgalConfig(warmup_ms=0.0))
        self.keys: Dict[int, List[int]] = {}       # swapped-out sequence -> its page keys, logical order
        self._next_key = 1
        self.stats = {"swapped_out_seqs": 0, "swapped_in_seqs": 0, "pages_out": 0, "pages_in": 0, "to_nvme": 0,
                      "packed_seqs": 0, "packed_pages": 0, "unpacked_pages": 0}

    # ---- who leaves ----------------------------------------------------------------------------------
    def _now_ms(self) -> float:
        return time.perf_counter() * 1e3

    def track(self, seq_id: int, pinned: bool = False):
        """A sequence entered the running set: one eviction group (a sequence's pages leave together)."""
        if seq_id in self.hgal.groups:
            return
        page = UnifiedVirtualPage(vpid=seq_id, kind=PayloadKind.KV, owner=seq_id)
        page.pinned = pinned
        self.hgal.add_page(page, group=seq_id, now_ms=self._now_ms())

    def touch(self, seq_ids):
        now = self._now_ms()
        for sid in seq_ids:
            if sid in self.hgal.groups:
                self.hgal.touch_group(sid, now)

    def forget(self, seq_id: int):
        self.hgal.remove_group(seq_id)

    def victim_order(self, running_ids) -> List[int]:
        """Running sequences, best victim first (idle, rarely touched, unpinned groups go first)."""
        now = self._now_ms()
        for sid in running_ids:
            self.track(sid)
        order = self.hgal.select_victims(1 << 30, now)
        live = set(running_ids)
        return [g for g in order if g in live]

    # ---- moving the bytes ----------------------------------------------------------------------------
    def _make_room_on_host(self, need: int):
        """Pinned host memory is the second tier: when it cannot take ``need`` more pages, the pages that have been
        there longest go down to the NVMe file (compressed, CRC-checked), as the reference's eviction worker does."""
        sw = self.swap
        if len(sw.host_free) >= need:
            return
        if sw.nvme is None:
            raise MemoryError(f"host swap space exhausted ({sw.host_pool.shape[0]} pages) and no NVMe tier configured")
        in_dram = sorted(((r.age, k) for k, r in sw.records.items() if r.tier == StorageTier.DRAM), reverse=True)
        for _, key in in_dram:
            if len(sw.host_free) >= need:
                break
            sw.execute(DmaCommand.EVICT_TO_NVME, key)
            self.stats["to_nvme"] += 1
        if len(sw.host_free) < need:
            raise MemoryError("swap space exhausted on both the host and the NVMe tier")

    def swap_out(self, item):
        """Copy the pages of a preempted sequence to the host (before the step's kernels may reuse them); with a
        device tier they are packed to 4 bits in place of the copy while the pool has room."""
        from ..kv_cache.header import PrecisionTier
        tier = self.tier_policy(int(item.seq_id)) if self.tier_policy is not None else PrecisionTier.KIVI4
        if self.device_tier is not None and tier >= PrecisionTier.KIVI4:
            pages = [int(p) for p in item.pages]
            # which pages keep full precision (host path): the sink pages, and with page telemetry those the KV optimiser
            # wants above 4 bits (page_tier(page) -> PrecisionTier, from the page headers)
            lossless = [j < self.sink_pages or (self.page_tier is not None and self.page_tier(pg) < PrecisionTier.KIVI4)
                        for j, pg in enumerate(pages)]
            slots = self.device_tier.pack([pg for pg, keep in zip(pages, lossless) if not keep])
            if slots is not None:
                n_host = sum(lossless)
                keys = []
                if n_host:
                    self._make_room_on_host(n_host)
                    for pg in (pg for pg, keep in zip(pages, lossless) if keep):
                        key = self._next_key
                        self._next_key += 1
                        self.swap.register(key, pg)
                        self.swap.execute(DmaCommand.EVICT_TO_DRAM, key)
                        keys.append(key)
                    self.swap.tick()
                ki, si = iter(keys), iter(slots)
                self.layout[int(item.seq_id)] = [("host", next(ki)) if keep else ("pool", next(si)) for keep in lossless]
                self.sink_keys[int(item.seq_id)] = keys
                self.packed[int(item.seq_id)] = slots
                self.forget(int(item.seq_id))
                self.stats["swapped_out_seqs"] += 1
                self.stats["packed_seqs"] += 1
                self.stats["packed_pages"] += len(slots)
                self.stats["pages_out"] += len(keys)
                return
        self._make_room_on_host(len(item.pages))
        keys = []
        for page in item.pages:
            key = self._next_key
            self._next_key += 1
            self.swap.register(key, int(page))
            self.swap.execute(DmaCommand.EVICT_TO_DRAM, key)
            keys.append(key)
        self.swap.tick()
        self.keys[int(item.seq_id)] = keys
        self.forget(int(item.seq_id))
        self.stats["swapped_out_seqs"] += 1
        self.stats["pages_out"] += len(keys)

    def swap_in(self, item):
        """Bring a sequence back into the pages the batcher just gave it (the last page may be a fresh, empty one)."""
        slots = self.packed.pop(int(item.seq_id), None)
        if slots is not None:
            pages = [int(p) for p in item.pages]
            layout = self.layout.pop(int(item.seq_id))
            self.sink_keys.pop(int(item.seq_id), None)
            pool_slots, pool_pages = [], []
            for (kind, ref), page in zip(layout, pages):       # logical order: entry j goes to the j-th new page
                if kind == "host":
                    if self.swap.records[ref].tier == StorageTier.NVME:
                        self._make_room_on_host(1)
                    self.swap.execute(DmaCommand.PROMOTE_TO_HBM, ref, dev_page=page)
                    del self.swap.records[ref]
                    self.stats["pages_in"] += 1
                else:
                    pool_slots.append(ref)
                    pool_pages.append(page)
            self.swap.dev_free.clear()
            self.device_tier.unpack(pool_slots, pool_pages)
            self.track(int(item.seq_id))
            self.stats["swapped_in_seqs"] += 1
            self.stats["unpacked_pages"] += len(pool_slots)
            return
        keys = self.keys.pop(int(item.seq_id), [])
        pairs = list(zip(keys, item.pages))
        # pages still in host memory first (each frees a host slot), then the ones that went down to the file tier:
        # those come up in two hops and need one free host slot on their way
        for tier in (StorageTier.DRAM, StorageTier.NVME):
            for key, page in pairs:
                if self.swap.records[key].tier != tier:
                    continue
                if tier == StorageTier.NVME:
                    self._make_room_on_host(1)
                self.swap.execute(DmaCommand.PROMOTE_TO_HBM, key, dev_page=int(page))
        for key in keys:
            del self.swap.records[key]
        self.swap.dev_free.clear()          # device pages belong to the batcher's allocator, not to the swap tier
        self.track(int(item.seq_id))
        self.stats["swapped_in_seqs"] += 1
        self.stats["pages_in"] += len(keys)

    def drop(self, seq_id: int):
        """A swapped-out sequence was aborted: release its copies."""
        slots = self.packed.pop(int(seq_id), None)
        if slots is not None:
            self.device_tier.release(slots)
            self.layout.pop(int(seq_id), None)
            self.keys[int(seq_id)] = self.sink_keys.pop(int(seq_id), [])      # released with the host copies below
        for key in self.keys.pop(int(seq_id), []):
            r = self.swap.records.pop(key, None)
            if r is None:
                continue
            if r.tier == StorageTier.DRAM:
                self.swap.host_free.append(r.location)
            elif r.tier == StorageTier.NVME and self.swap.nvme is not None:
                self.swap.nvme.free.append(r.location)

    def close(self):
        self.swap.close()
