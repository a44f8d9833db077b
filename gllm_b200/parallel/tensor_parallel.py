"""Tensor parallelism over NVLink/NVSwitch: one process per GPU, activations replicated, weights sharded
(column-parallel q/k/v/gate/up/lm_head, row-parallel o_proj/down_proj).

The reference does every TP collective on host f32 slices through its NCCL wrapper
(src/engine/coordinator/compute.rs:122-436: tp_all_reduce / tp_reduce_scatter / tp_all_gather,
src/engine/distributed_config.rs:424-495). Here the row-parallel GEMM and its all-reduce are ONE kernel
(``gllm_gemm_bf16_residual_allreduce``): each rank stores its bf16 partial tiles into its own symmetric
buffer as the tcgen05 tiles retire, all CTAs of all ranks meet at an arrival counter, and every rank then
pulls the sum of all partials — one ``multimem.ld_reduce`` per 16 bytes, added in fp32 inside NVSwitch, when
the buffer has a multicast mapping, otherwise plain peer loads over NVLink — and finishes locally (residual
add, bf16 store, next norm's row statistics). Bulk data never goes through atomics: accumulating partial
tiles with ``red``/``multimem.red`` was measured at roughly 20x the time of this pull design. The NCCL path (unfused GEMM -> ncclAllReduce -> residual/norm-stat kernel) is kept as the
selectable baseline.

Modes: ``fused`` (multimem if available, else peer loads), ``fused_p2p`` (force peer loads), ``nccl``,
``auto`` (fused when symmetric memory can be set up, else nccl).
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from .. import ops
from ..ops import _native as nv


class TPContext:
    def __init__(self, rank: int, size: int, device, *, mode: str = "auto", max_tokens: int = 1024, hidden: int = 4096,
                 group=None, max_fused_tokens: int = 1024):
        self.rank, self.size, self.device = rank, size, torch.device(device)
        self.group = group
        self.requested_mode = mode
        self.mode = "nccl"
        self.uses_multimem = False
        self.max_fused_tokens = min(max_fused_tokens, max_tokens)
        self.fused_max_k = 1 << 30      # `auto` mode: longest local K that still takes the fused kernel
        self.n_pad = ((hidden + 255) // 256) * 256
        self.buf_elems = self.max_fused_tokens * self.n_pad
        self._symm = None
        self._handle = None
        if mode in ("auto", "fused", "fused_p2p") and self.device.type == "cuda":
            try:
                self._setup_symmetric(force_p2p=(mode == "fused_p2p"))
                self.mode = "fused"
            except Exception as exc:  # no NVLink peer access / symmetric memory unavailable
                if mode != "auto":
                    raise
                self.setup_error = repr(exc)
                self.mode = "nccl"

    # ------------------------------------------------------------------------------------------
    def _setup_symmetric(self, force_p2p: bool):
        import torch.distributed as dist
        total = 3 * self.buf_elems + 64     # two alternating partial buffers, the two-shot result region, counters
        if self.size == 1:
            buf = torch.zeros(total, dtype=torch.bfloat16, device=self.device)
            peer_ptrs, mc_ptr = [buf.data_ptr()], 0
        else:
            import torch.distributed._symmetric_memory as symm_mem
            group = self.group or dist.group.WORLD
            buf = symm_mem.empty(total, dtype=torch.bfloat16, device=self.device)
            self._handle = symm_mem.rendezvous(buf, group.group_name)
            buf.zero_()
            torch.cuda.synchronize(self.device)
            dist.barrier(group=group)
            peer_ptrs = [int(p) for p in self._handle.buffer_ptrs]
            mc_ptr = 0 if force_p2p else int(getattr(self._handle, "multicast_ptr", 0) or 0)
        self._symm = buf
        self.uses_multimem = mc_ptr != 0
        counter_off = 3 * self.buf_elems * 2  # bytes; 8-byte aligned because buf_elems is a multiple of 256
        n = len(peer_ptrs)
        self._peer_acc = (ctypes.c_void_p * 8)(*([p for p in peer_ptrs] + [None] * (8 - n)))
        self._peer_cnt = (ctypes.c_void_p * 8)(*([p + counter_off for p in peer_ptrs] + [None] * (8 - n)))
        self._mc_acc = mc_ptr or None
        self._mc_cnt = (mc_ptr + counter_off) if mc_ptr else None
        self._state = torch.zeros(8, dtype=torch.int64, device=self.device)

    # ------------------------------------------------------------------------------------------
    def gemm_allreduce_residual(self, a, w, x, ss_out, partial, *, bn: int = 256):
        """x <- sum_ranks(a @ w.T) + x ; returns the tensor holding the row statistics of the new x."""
        M, K = a.shape
        N = w.shape[0]
        # The fused kernel publishes one partial per tile (no split of K inside the rank). Measured on B200 at
        # Qwen3-8B shapes, decode batch 256 (tokens/s fused vs unfused GEMM + NCCL all-reduce): 2 ranks 21.8k vs
        # 20.1k, 4 ranks 28.5k vs 25.6k, 8 ranks 31.6k vs 27.8k: fused is ahead everywhere, so `auto` always takes
        # it; `fused_max_k` stays as a knob.
        k_ok = self.requested_mode != "auto" or K <= self.fused_max_k
        if self.mode == "fused" and k_ok and M <= self.max_fused_tokens and N <= self.n_pad:
            parts = (N + 255) // 256  # the fused kernel reports statistics per 256-column group
            ss = ss_out[:M, :parts]
            if not ss.is_contiguous():
                raise ValueError("row statistics buffer must be [tokens, parts] contiguous")
            # few output tiles: prefer 128-wide tiles so more SMs stream weights (the pull phase works on
            # 256-column groups either way)
            tile_bn = 256 if (N // 256) * ((M + 127) // 128) >= 148 else 128
            rc = nv.lib().gllm_gemm_bf16_residual_allreduce(
                a.data_ptr(), a.stride(0), w.data_ptr(), w.stride(0), x.data_ptr(), x.stride(0), x.data_ptr(),
                x.stride(0), ss.data_ptr(), M, N, K, None, tile_bn, nv.stream_ptr(), 0, 0, self.size, self.rank,
                self._mc_acc, ctypes.cast(self._peer_acc, ctypes.c_void_p), self._mc_cnt,
                ctypes.cast(self._peer_cnt, ctypes.c_void_p), self._state.data_ptr(), self.buf_elems)
            nv.check(rc, "gemm_bf16_residual_allreduce")
            return ss
        # NCCL baseline: unfused GEMM -> all-reduce -> residual add + row statistics
        import torch.distributed as dist
        p = partial[:M]
        ops.gemm(a, w, out=p, bn=bn)
        if self.size > 1:
            dist.all_reduce(p, group=self.group)
        ss = ss_out.reshape(-1)[:M].view(M, 1)
        ops.rmsnorm(p, None, 0.0, residual=x, h_out=x, ss_out=ss, want_y=False)
        return ss

    # ------------------------------------------------------------------------------------------
    def sample_vocab_parallel(self, logits, vocab_local, vocab_start, params, seed, offsets, out, vocab, greedy=True):
        """Each rank holds logits for vocabulary rows [vocab_start, vocab_start+vocab_local). Greedy requests
        exchange only (max, argmax) pairs; otherwise the shards are gathered and sampled identically on every
        rank (same Philox seed and offsets), so all ranks agree on the token without another broadcast."""
        import torch.distributed as dist
        B = logits.shape[0]
        if greedy:
            vals = torch.empty(B, dtype=torch.float32, device=logits.device)
            idx = torch.empty(B, dtype=torch.int32, device=logits.device)
            ops.argmax(logits, vocab_local, out=idx, out_vals=vals)
            pair = torch.stack([vals, (idx + vocab_start).to(torch.float32)], 1).contiguous()
            allp = torch.empty((self.size, B, 2), dtype=torch.float32, device=logits.device)
            dist.all_gather_into_tensor(allp, pair, group=self.group)
            best = allp[:, :, 0].argmax(0)  # first rank wins ties -> lowest vocabulary index
            out.copy_(allp[best, torch.arange(B, device=logits.device), 1].to(torch.int32))
            return out
        shard = logits[:, :vocab_local].contiguous()
        # shards may differ by one row when vocab % size != 0: pad to the widest
        width = (vocab + self.size - 1) // self.size
        if shard.shape[1] < width:
            shard = torch.nn.functional.pad(shard, (0, width - shard.shape[1]), value=float("-inf"))
        allv = torch.empty((self.size, B, width), dtype=torch.float32, device=logits.device)
        dist.all_gather_into_tensor(allv, shard, group=self.group)
        full = allv.permute(1, 0, 2).reshape(B, self.size * width)
        if self.size * width != vocab:
            from ..models.weights import shard_range
            cols = torch.cat([torch.arange(self.size * 0 + r * width, r * width + (shard_range(vocab, r, self.size)[1] -
                                                                                  shard_range(vocab, r, self.size)[0]),
                                           device=logits.device) for r in range(self.size)])
            full = full.index_select(1, cols)
        return ops.sample(full.contiguous(), params, vocab=vocab, seed=seed, step_offsets=offsets, out=out)

    def close(self):
        self._symm = None
        self._handle = None


def single_gpu_context(device, hidden: int, max_tokens: int = 1024) -> TPContext:
    """A world-size-1 context on ordinary device memory: exercises the fused kernel's protocol (alternating
    buffers, arrival counter, launch state) on one GPU."""
    return TPContext(0, 1, device, mode="fused_p2p", max_tokens=max_tokens, hidden=hidden)
