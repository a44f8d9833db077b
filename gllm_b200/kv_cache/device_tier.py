"""Device-side 4-bit KV tier: whole KV pages packed into a byte pool on the GPU (KIVI layout: keys per channel,
values per token), unpacked back into bf16 pages, or read in place by the tiered attention kernel.

CUDA path: ``csrc/kernels/kv_tier.cu``. CPU path / oracle: the same arithmetic in PyTorch (fp16-rounded scale and
zero, nearest code), so packed bytes made on either side unpack on the other.

A cache page is ``[2, n_kv, 16, D]`` bf16; its packed form takes ``n_kv * (20 * D + 64)`` bytes (for D = 128: 2624 per
head against 8192): per head ``[K codes 8D | K scale D fp16 | K zero D fp16 | V codes 8D | V scale 16 fp16 | V zero 16
fp16]``, two codes per byte, even channel in the low nibble.

Reference parity: KIVI quantisation of cold pages and per-page precision tiers
(src/kv_cache/quant.rs:35-700, src/scheduler/kv_optimizer.rs:131-192,446-830).
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch

from ..ops import _native as nv
from ..ops._native import F, I, L, P

nv.register("gllm_kivi4_page_bytes", L, [I, I])
nv.register("gllm_kivi4_pack_pages", I, [P, I, P, I, P, P, I, I, I, P])
nv.register("gllm_kivi4_unpack_pages", I, [P, I, P, I, P, P, I, I, I, P])
nv.register("gllm_paged_attention_tiered", I, [P, P, P, I, P, I, P, I, P, P, P, I, I, I, I, I, F, I, I, P])


def page_bytes(n_kv: int, head_dim: int) -> int:
    return n_kv * (20 * head_dim + 64)


def _geometry(cache: torch.Tensor):
    if cache.dim() != 5 or cache.shape[1] != 2 or cache.shape[3] != 16:
        raise ValueError(f"KV cache must be [pages, 2, n_kv, 16, D], got {tuple(cache.shape)}")
    return int(cache.shape[2]), int(cache.shape[4])


def _range(lo, hi):
    """(scale, zero) as the reader sees them: rounded to fp16, a zero scale replaced by 1."""
    s = ((hi - lo) / 15.0).to(torch.float16)
    z = lo.to(torch.float16)
    sf = s.float()
    return s, z, torch.where(sf > 0, sf, torch.ones_like(sf)), z.float()


def _pack_ref(pages: torch.Tensor) -> torch.Tensor:
    """pages [n, 2, n_kv, 16, D] (any float dtype) -> bytes [n, page_bytes]."""
    n, _, n_kv, _, D = pages.shape
    x = pages.float()
    out = torch.zeros((n, n_kv, 20 * D + 64), dtype=torch.uint8, device=pages.device)

    def nibbles(codes):      # [..., 16, D] -> [..., 16 * D / 2]
        c = codes.to(torch.int32)
        return (c[..., 0::2] | (c[..., 1::2] << 4)).to(torch.uint8).reshape(*codes.shape[:-2], -1)

    k, v = x[:, 0], x[:, 1]                                   # [n, n_kv, 16, D]
    ks16, kz16, ks, kz = _range(k.amin(2), k.amax(2))         # per channel: [n, n_kv, D]
    kc = torch.round((k - kz[:, :, None, :]) / ks[:, :, None, :]).clamp_(0, 15)
    vs16, vz16, vs, vz = _range(v.amin(3), v.amax(3))         # per token: [n, n_kv, 16]
    vc = torch.round((v - vz[..., None]) / vs[..., None]).clamp_(0, 15)
    out[:, :, :8 * D] = nibbles(kc)
    out[:, :, 8 * D:10 * D] = ks16.view(torch.uint8).reshape(n, n_kv, 2 * D)
    out[:, :, 10 * D:12 * D] = kz16.view(torch.uint8).reshape(n, n_kv, 2 * D)
    out[:, :, 12 * D:20 * D] = nibbles(vc)
    out[:, :, 20 * D:20 * D + 32] = vs16.view(torch.uint8).reshape(n, n_kv, 32)
    out[:, :, 20 * D + 32:] = vz16.view(torch.uint8).reshape(n, n_kv, 32)
    return out.reshape(n, -1)


def _unpack_ref(packed: torch.Tensor, n_kv: int, D: int) -> torch.Tensor:
    """bytes [n, page_bytes] -> fp32 pages [n, 2, n_kv, 16, D]."""
    n = packed.shape[0]
    b = packed.reshape(n, n_kv, 20 * D + 64)

    def codes(x):            # [n, n_kv, 8D] -> [n, n_kv, 16, D]
        c = x.to(torch.int32)
        return torch.stack([c & 15, c >> 4], -1).reshape(n, n_kv, 16, D).float()

    def halves(x, count):
        s = x.contiguous().view(torch.float16).reshape(n, n_kv, count).float()
        return s

    ks = halves(b[:, :, 8 * D:10 * D], D)
    ks = torch.where(ks > 0, ks, torch.ones_like(ks))
    kz = halves(b[:, :, 10 * D:12 * D], D)
    vs = halves(b[:, :, 20 * D:20 * D + 32], 16)
    vs = torch.where(vs > 0, vs, torch.ones_like(vs))
    vz = halves(b[:, :, 20 * D + 32:], 16)
    k = codes(b[:, :, :8 * D]) * ks[:, :, None, :] + kz[:, :, None, :]
    v = codes(b[:, :, 12 * D:20 * D]) * vs[..., None] + vz[..., None]
    return torch.stack([k, v], 1)


def _ids(x, device) -> torch.Tensor:
    return torch.as_tensor(x, dtype=torch.int32, device=device).contiguous()


def pack_pages(cache: torch.Tensor, pool: torch.Tensor, page_ids, slots) -> None:
    """pool[slots[i]] <- packed form of cache[page_ids[i]] (one layer)."""
    n_kv, D = _geometry(cache)
    page_ids, slots = _ids(page_ids, cache.device), _ids(slots, cache.device)
    if page_ids.numel() == 0:
        return
    if not cache.is_cuda:
        pool[slots.long()] = _pack_ref(cache[page_ids.long()])
        return
    if cache.dtype != torch.bfloat16:
        raise ValueError("the packing kernel reads bf16 pages")
    rc = nv.lib().gllm_kivi4_pack_pages(cache.data_ptr(), cache.shape[0], pool.data_ptr(), pool.shape[0], page_ids.data_ptr(),
                                        slots.data_ptr(), page_ids.numel(), n_kv, D, nv.stream_ptr())
    nv.check(rc, "kivi4_pack_pages")


def unpack_pages(cache: torch.Tensor, pool: torch.Tensor, slots, page_ids) -> None:
    """cache[page_ids[i]] <- pool[slots[i]] dequantised (one layer)."""
    n_kv, D = _geometry(cache)
    page_ids, slots = _ids(page_ids, cache.device), _ids(slots, cache.device)
    if page_ids.numel() == 0:
        return
    if not cache.is_cuda:
        cache[page_ids.long()] = _unpack_ref(pool[slots.long()], n_kv, D).to(cache.dtype)
        return
    rc = nv.lib().gllm_kivi4_unpack_pages(cache.data_ptr(), cache.shape[0], pool.data_ptr(), pool.shape[0], slots.data_ptr(),
                                          page_ids.data_ptr(), page_ids.numel(), n_kv, D, nv.stream_ptr())
    nv.check(rc, "kivi4_unpack_pages")


def paged_attention_tiered(q, cache, pool, block_tables, q_start, q_len, ctx_lens, *, max_q_len, n_q, n_kv, scale,
                           causal=True, window=0, out=None):
    """Attention over block tables that mix tiers: entry p >= 0 is bf16 page p of ``cache``, entry p < 0 is slot
    ``-p - 1`` of ``pool``, dequantised while it is read. q [T, n_q * D] -> [T, n_q * D]."""
    n_kv_c, D = _geometry(cache)
    if out is None:
        out = torch.empty_like(q)
    if not q.is_cuda:
        from ..ops.attention import attention_ref
        # oracle: unpack every referenced slot into scratch pages behind the cache, then the plain reference
        bt = block_tables.clone().long()
        neg = bt < 0
        slots = torch.unique((-bt[neg] - 1))
        scratch = _unpack_ref(pool[slots], n_kv, D).to(cache.dtype) if slots.numel() else cache[:0]
        remap = {int(s): cache.shape[0] + i for i, s in enumerate(slots.tolist())}
        bt2 = bt.clone()
        for idx in neg.nonzero().tolist():
            bt2[idx[0], idx[1]] = remap[int(-bt[idx[0], idx[1]] - 1)]
        both = torch.cat([cache, scratch], 0)
        out.copy_(attention_ref(q, both, bt2.to(torch.int32), q_start, q_len, ctx_lens, n_q, n_kv, scale, causal, window, None))
        return out
    rc = nv.lib().gllm_paged_attention_tiered(q.data_ptr(), out.data_ptr(), cache.data_ptr(), cache.shape[0], pool.data_ptr(),
                                              pool.shape[0], block_tables.data_ptr(), block_tables.shape[1],
                                              q_start.data_ptr(), q_len.data_ptr(), ctx_lens.data_ptr(), q_len.shape[0],
                                              int(max_q_len), n_q, n_kv, D, float(scale), 1 if causal else 0, int(window),
                                              nv.stream_ptr())
    nv.check(rc, "paged_attention_tiered")
    return out


class Kivi4Pool:
    """The packed tier of a whole model: one byte pool per layer, one slot index shared by all layers (slot s of every
    layer holds the same logical page, as page p does in the bf16 caches)."""

    def __init__(self, kv_caches: Sequence[torch.Tensor], pool_pages: int):
        self.n_kv, self.head_dim = _geometry(kv_caches[0])
        self.page_bytes = page_bytes(self.n_kv, self.head_dim)
        seen = {}
        self.pools: List[torch.Tensor] = []
        for c in kv_caches:      # shared-KV layers alias their donor's cache: they share its pool too
            key = c.data_ptr()
            if key not in seen:
                seen[key] = torch.zeros((pool_pages, self.page_bytes), dtype=torch.uint8, device=c.device)
            self.pools.append(seen[key])
        self._unique = list(seen.items())
        self._caches = {c.data_ptr(): c for c in kv_caches}
        self.free: List[int] = list(range(pool_pages - 1, -1, -1))
        self.capacity = pool_pages

    @property
    def bytes_per_page_all_layers(self) -> int:
        return self.page_bytes * len(self._unique)

    def pack(self, page_ids: Sequence[int]) -> Optional[List[int]]:
        """Pack these pages of every layer; returns their slots, or None when the pool has not enough free slots."""
        if len(page_ids) > len(self.free):
            return None
        slots = [self.free.pop() for _ in page_ids]
        for ptr, pool in self._unique:
            pack_pages(self._caches[ptr], pool, list(page_ids), slots)
        return slots

    def unpack(self, slots: Sequence[int], page_ids: Sequence[int]) -> None:
        """Dequantise the slots into these pages of every layer and release the slots."""
        for ptr, pool in self._unique:
            unpack_pages(self._caches[ptr], pool, list(slots), list(page_ids))
        self.release(slots)

    def release(self, slots: Sequence[int]) -> None:
        self.free.extend(int(s) for s in slots)
