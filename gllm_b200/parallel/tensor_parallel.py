"""Tensor parallelism over NVLink/NVSwitch: one process per GPU, activations replicated, weights sharded
(column-parallel q/k/v/gate/up/lm_head, row-parallel o_proj/down_proj).

The reference does every TP collective on host f32 slices through its NCCL wrapper
(src/engine/coordinator/compute.rs:122-436: tp_all_reduce / tp_reduce_scatter / tp_all_gather,
src/engine/distributed_config.rs:424-495). Here the row-parallel GEMM and its all-reduce are ONE kernel, in two
forms:

``push`` (default, ``gllm_gemm_bf16_residual_allreduce_push``): rank r owns the output rows
[r * ceil(M/W), ...). As each tcgen05 tile retires, its bf16 rows are stored straight into the owner's receive
slots with peer stores over NVLink and a per-tile flag is released; the owner's warps wait tile by tile (no meeting
of all ranks before data moves), add the sources in a fixed order, add the residual and store the finished rows and
their norm statistics into EVERY rank's activation buffer (one ``multimem.st`` per 16 bytes through NVSwitch, or a
store per peer). The activation buffer ``x`` and the statistics therefore live inside the symmetric region
(``workspace_buffers``); a caller's ordinary tensor is staged through it. The kernel ends with one exchange of
per-rank "done" words.

``ll`` (``gllm_gemm_bf16_residual_allreduce_ll``, decode-sized M): the same ownership of rows, but no flags, fences
or meetings at all. Every 32-bit word of the receive and result slots is either the sentinel 0x80008000 (a pair of
bf16 negative zeros, which the writers replace by +0) or data; readers poll the data words themselves and put the
sentinel back after reading, and two parity sets of slots alternate between launches. The finished rows go into
every rank's result slots and each rank copies them into its ordinary activation tensor, computing the norm
statistics on the way. At decode sizes every CTA holds one 128-wide tile (parked in shared memory, K split inside the
rank); at prefill sizes the CTAs run several 256-wide tiles and their epilogue warps store the rows as the tiles
retire, the reduce and gather phases follow the tile loop.

``pull`` (``gllm_gemm_bf16_residual_allreduce``): every rank stores its partial tiles in its own symmetric buffer,
all ranks meet at an arrival counter, and every rank pulls the sum (``multimem.ld_reduce`` or peer loads), one-shot
or two-shot. Kept for comparison.

The NCCL path (unfused GEMM -> ncclAllReduce -> residual/norm-stat kernel) is the selectable baseline.

Modes: ``auto`` (the fused form that measured fastest when symmetric memory can be set up, else nccl), ``ll`` /
``ll_p2p`` (low-latency form at decode sizes, push above), ``fused`` (push; multimem if available), ``fused_p2p``
(push, peer stores only), ``pull`` / ``pull_p2p``, ``nccl``.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from .. import ops
from ..ops import _native as nv

_FLAG_COUNT = 32768      # u32 tile flags of the push form
_LL_SENTINEL = -2147450880   # 0x80008000 as int32: "no data yet" in the slots of the low-latency form
_AUTO_FORM = "ll"


def _align(n: int, a: int = 256) -> int:
    return (n + a - 1) // a * a


class TPContext:
    def __init__(self, rank: int, size: int, device, *, mode: str = "auto", max_tokens: int = 1024, hidden: int = 4096,
                 group=None, max_fused_tokens: Optional[int] = None):
        self.rank, self.size, self.device = rank, size, torch.device(device)
        self.group = group
        self.requested_mode = mode
        self.mode = "nccl"
        self.form = "none"            # "ll" | "push" | "pull" once the fused kernel is set up
        self.ll_max_tokens = max_tokens          # the low-latency form takes every M the context was sized for
        self.ag_max_tokens = min(1024, max_tokens)
        self.uses_multimem = False
        self.max_tokens = max_tokens
        self.hidden = hidden
        # pull form: its three buffers are sized for decode batches only
        self.max_fused_tokens = min(max_fused_tokens or (1024 if mode.startswith("pull") else max_tokens), max_tokens)
        self.fused_max_k = 1 << 30      # `auto` mode: longest local K that still takes the fused kernel
        self.n_pad = ((hidden + 255) // 256) * 256
        self.buf_elems = self.max_fused_tokens * self.n_pad
        self._symm = None
        self._handle = None
        self.baseline = False           # True: run the NCCL path although the fused one is set up (bench baseline arm)
        if mode in ("auto", "ll", "ll_p2p", "fused", "fused_p2p", "pull", "pull_p2p") and self.device.type == "cuda":
            try:
                self.form = ("pull" if mode.startswith("pull") else "ll" if mode.startswith("ll") else
                             _AUTO_FORM if mode == "auto" else "push")
                self._setup_symmetric(force_p2p=mode.endswith("_p2p"))
                self.mode = "fused"
            except Exception as exc:  # no NVLink peer access / symmetric memory unavailable
                if mode != "auto":
                    raise
                self.setup_error = repr(exc)
                self.mode, self.form = "nccl", "none"

    # ------------------------------------------------------------------------------------------
    def _layout(self):
        """Byte offsets of the regions inside the symmetric allocation (identical on every rank)."""
        T, W = self.max_tokens, self.size
        parts = (self.hidden + 127) // 128
        off, lay = 0, {}

        def take(name, nbytes):
            nonlocal off
            lay[name] = (off, nbytes)
            off = _align(off + nbytes)
        if self.form == "push":
            recv_rows = max(T + 8, min(4 * (T + 8), 4160))     # room for K splits inside a rank at decode sizes
            take("recv", recv_rows * self.n_pad * 2)
            take("x", T * self.hidden * 2)
            for name in ("ss0", "ss_a", "ss_b", "ss_stage"):
                take(name, T * parts * 4)
            take("flags", _FLAG_COUNT * 4)
            take("done", 64)
        elif self.form == "ll":
            # one parity set of receive slots: every rank's partial rows, times up to four K splits at decode sizes
            # (one split at prefill sizes); one parity set of result slots: all finished rows
            recv_rows = max(4 * (min(T, 1024) + 8), T + 8)
            self._ll_recv_bytes = _align(recv_rows * self.n_pad * 2)
            self._ll_res_bytes = _align(T * self.n_pad * 2)
            take("ll_recv", 2 * self._ll_recv_bytes)
            take("ll_res", 2 * self._ll_res_bytes)
            # slots of the all-gather in front of a column-parallel GEMM (sequence-parallel activations)
            self._ag_bytes = _align(self.ag_max_tokens * self.n_pad * 2)
            take("ag_slots", 2 * self._ag_bytes)
        else:
            take("pull", 3 * self.buf_elems * 2)
            take("counters", 64)
        lay["_total"] = (off, 0)
        return lay

    def _setup_symmetric(self, force_p2p: bool):
        import torch.distributed as dist
        lay = self._layout()
        total = lay["_total"][0]
        if self.size == 1:
            buf = torch.zeros(total, dtype=torch.uint8, device=self.device)
            self._symm, self._lay = buf, lay
            self._fill_sentinel()
            peer_ptrs, mc_ptr = [buf.data_ptr()], 0
        else:
            import torch.distributed._symmetric_memory as symm_mem
            group = self.group or dist.group.WORLD
            buf = symm_mem.empty(total, dtype=torch.uint8, device=self.device)
            self._handle = symm_mem.rendezvous(buf, group.group_name)
            buf.zero_()
            self._symm, self._lay = buf, lay
            self._fill_sentinel()
            torch.cuda.synchronize(self.device)
            dist.barrier(group=group)
            peer_ptrs = [int(p) for p in self._handle.buffer_ptrs]
            mc_ptr = 0 if force_p2p else int(getattr(self._handle, "multicast_ptr", 0) or 0)
        self._symm, self._lay, self._total = buf, lay, total
        self._base = buf.data_ptr()
        self.uses_multimem = mc_ptr != 0
        n = len(peer_ptrs)
        self._mc_base = mc_ptr or None
        self._peer_base = (ctypes.c_void_p * 8)(*([p for p in peer_ptrs] + [None] * (8 - n)))
        self._state = torch.zeros(8, dtype=torch.int64, device=self.device)
        self._ag_state = torch.zeros(8, dtype=torch.int64, device=self.device)
        self._sms = int(nv.lib().gllm_sm_count())
        if self.form == "pull":
            off = lay["pull"][0]
            counter_off = off + 3 * self.buf_elems * 2
            self._peer_acc = (ctypes.c_void_p * 8)(*([p + off for p in peer_ptrs] + [None] * (8 - n)))
            self._peer_cnt = (ctypes.c_void_p * 8)(*([p + counter_off for p in peer_ptrs] + [None] * (8 - n)))
            self._mc_acc = (mc_ptr + off) if mc_ptr else None
            self._mc_cnt = (mc_ptr + counter_off) if mc_ptr else None

    def _fill_sentinel(self):
        for name in ("ll_recv", "ll_res", "ag_slots"):
            if name in self._lay:
                off, nbytes = self._lay[name]
                self._symm[off:off + nbytes].view(torch.int32).fill_(_LL_SENTINEL)

    def _view(self, name, dtype, shape):
        off, nbytes = self._lay[name]
        n = 1
        for d in shape:
            n *= d
        return self._symm[off:off + n * torch.empty(0, dtype=dtype).element_size()].view(dtype).view(*shape)

    def workspace_buffers(self, tokens: int):
        """Activation buffer and norm-statistics buffers inside the symmetric region, for a model whose residual
        stream the push kernel updates on every rank. None when the push form is not in use or ``tokens`` exceeds
        what the region was sized for."""
        if self.mode != "fused" or self.form != "push" or tokens > self.max_tokens:
            return None
        parts = (self.hidden + 127) // 128
        return dict(x=self._view("x", torch.bfloat16, (self.max_tokens, self.hidden))[:tokens],
                    ss0=self._view("ss0", torch.float32, (self.max_tokens, parts))[:tokens],
                    ss_a=self._view("ss_a", torch.float32, (self.max_tokens, parts))[:tokens],
                    ss_b=self._view("ss_b", torch.float32, (self.max_tokens, parts))[:tokens])

    def _inside(self, t) -> bool:
        return self._base <= t.data_ptr() and t.data_ptr() + t.numel() * t.element_size() <= self._base + self._total

    # ------------------------------------------------------------------------------------------
    def gemm_allreduce_residual(self, a, w, x, ss_out, partial, *, bn: int = 256):
        """x <- sum_ranks(a @ w.T) + x ; returns the tensor holding the row statistics of the new x."""
        M, K = a.shape
        N = w.shape[0]
        k_ok = self.requested_mode != "auto" or K <= self.fused_max_k
        fused = self.mode == "fused" and not self.baseline and k_ok and N <= self.n_pad
        if fused and self.form == "ll" and M <= self.ll_max_tokens and x.stride(0) * 2 % 16 == 0:
            parts = (N + 255) // 256
            ss = ss_out[:M, :parts]
            if not ss.is_contiguous():
                raise ValueError("row statistics buffer must be [tokens, parts] contiguous")
            lay = self._lay
            # decode sizes: 128-wide tiles, one per CTA (parked in shared memory, local K split); prefill sizes: 256-wide
            # tiles, several per CTA, rows stored by the epilogue warps as the tiles retire
            one_per_cta = ((M + 127) // 128) * (self.n_pad // 128) <= self._sms
            rc = nv.lib().gllm_gemm_bf16_residual_allreduce_ll(
                a.data_ptr(), a.stride(0), w.data_ptr(), w.stride(0), x.data_ptr(), x.stride(0), ss.data_ptr(), M, N, K,
                None, 128 if one_per_cta or N % 256 else 256, nv.stream_ptr(), self.size, self.rank, self._mc_base, ctypes.cast(self._peer_base, ctypes.c_void_p),
                self._total, lay["ll_recv"][0], self._ll_recv_bytes, lay["ll_res"][0], self._ll_res_bytes, self._state.data_ptr())
            nv.check(rc, "gemm_bf16_residual_allreduce_ll")
            return ss
        if fused and self.form == "push" and M <= self.max_tokens and x.stride(0) * 2 % 16 == 0:
            parts = (N + 255) // 256  # the fused kernel reports statistics per 256-column group
            ss = ss_out[:M, :parts]
            if not ss.is_contiguous():
                raise ValueError("row statistics buffer must be [tokens, parts] contiguous")
            staged = not (self._inside(x) and self._inside(ss))
            xs, sss = x, ss
            if staged:      # a caller's ordinary tensors: run on the symmetric staging buffers
                xs = self._view("x", torch.bfloat16, (self.max_tokens, self.hidden))[:M, :N]
                xs.copy_(x)
                sss = self._view("ss_stage", torch.float32, (self.max_tokens * ((self.hidden + 127) // 128),))[:M * parts].view(M, parts)
            # few output tiles: 128-wide tiles so that more SMs stream weights
            tile_bn = 256 if (N // 256) * ((M + 127) // 128) >= 148 else 128
            lay = self._lay
            rc = nv.lib().gllm_gemm_bf16_residual_allreduce_push(
                a.data_ptr(), a.stride(0), w.data_ptr(), w.stride(0), xs.data_ptr(), xs.stride(0), sss.data_ptr(), M, N, K,
                None, tile_bn, nv.stream_ptr(), self.size, self.rank, self._mc_base,
                ctypes.cast(self._peer_base, ctypes.c_void_p), self._total, lay["recv"][0], lay["recv"][1] // 2,
                lay["flags"][0], _FLAG_COUNT, lay["done"][0], self._state.data_ptr())
            nv.check(rc, "gemm_bf16_residual_allreduce_push")
            if staged:
                x.copy_(xs)
                ss.copy_(sss)
            return ss
        if fused and self.form == "pull" and M <= self.max_fused_tokens:
            parts = (N + 255) // 256
            ss = ss_out[:M, :parts]
            if not ss.is_contiguous():
                raise ValueError("row statistics buffer must be [tokens, parts] contiguous")
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

    def can_fuse_blockscaled(self, M: int, N: int) -> bool:
        """Whether ``gemm_allreduce_residual_bs`` runs as one kernel for an [M, N] output."""
        return (self.mode == "fused" and self.form == "ll" and not self.baseline and M <= self.ll_max_tokens and
                N <= self.n_pad and N % 256 == 0)

    def gemm_allreduce_residual_bs(self, aq, w, x, ss_out):
        """Block-scaled (MXFP8 / NVFP4) row-parallel GEMM with the low-latency all-reduce in its epilogue:
        x <- sum_ranks(aq @ w.T) + x; returns the row statistics [M, ceil(N / 256)] of the new x. ``aq`` / ``w`` are
        ``ops.blockscale.BlockScaled`` operands. Callers check ``can_fuse_blockscaled`` first."""
        from ..ops import blockscale as B
        M, N = aq.rows, w.rows
        parts = (N + 255) // 256
        ss = ss_out.reshape(-1)[:M * parts].view(M, parts)
        one_per_cta = ((M + 127) // 128) * (self.n_pad // 128) <= self._sms
        lay = self._lay
        B.gemm_residual_allreduce(
            aq, w, x, ss, bn=128 if one_per_cta or N % 256 else 256, world=self.size, rank=self.rank,
            mc_base=self._mc_base, peer_base=ctypes.cast(self._peer_base, ctypes.c_void_p), region_bytes=self._total,
            recv_off=lay["ll_recv"][0], recv_bytes=self._ll_recv_bytes, res_off=lay["ll_res"][0],
            res_bytes=self._ll_res_bytes, state=self._state.data_ptr())
        return ss

    # ---- sequence-parallel forms: rows of the activations sharded over the ranks ----------------------------
    def shard_rows(self, M: int):
        """(first row, row count) of this rank's shard of an [M, ...] activation: rows [r * ceil(M / W), ...)."""
        per = (M + self.size - 1) // self.size
        lo = min(M, self.rank * per)
        return lo, min(M, lo + per) - lo

    def gemm_reduce_scatter_residual(self, a, w, x_shard, ss_out, M: int):
        """Row-parallel GEMM whose sum over ranks stays sharded by rows (reduce-scatter instead of all-reduce):
        x_shard <- rows of sum_ranks(a @ w.T) owned by this rank + x_shard. ``a`` [M, K_local], ``x_shard``
        [ceil(M / W), N] (the first ``shard_rows(M)[1]`` rows are used). One kernel in the low-latency form; unfused
        GEMM + all-reduce + slice otherwise. Reference: tp_reduce_scatter (src/engine/coordinator/compute.rs:148-164)."""
        K = a.shape[1]
        N = w.shape[0]
        lo, n_own = self.shard_rows(M)
        parts = (N + 255) // 256
        ss = ss_out[:max(n_own, 1), :parts]
        fused = (self.mode == "fused" and self.form == "ll" and not self.baseline and M <= min(self.ll_max_tokens, 1024) and
                 N <= self.n_pad and ((M + 127) // 128) * (self.n_pad // 128) <= self._sms and ss.is_contiguous())
        if fused:
            lay = self._lay
            rc = nv.lib().gllm_gemm_bf16_residual_reduce_scatter(
                a.data_ptr(), a.stride(0), w.data_ptr(), w.stride(0), x_shard.data_ptr(), x_shard.stride(0), ss.data_ptr(),
                M, N, K, None, nv.stream_ptr(), self.size, self.rank, ctypes.cast(self._peer_base, ctypes.c_void_p),
                self._total, lay["ll_recv"][0], self._ll_recv_bytes, self._state.data_ptr())
            nv.check(rc, "gemm_bf16_residual_reduce_scatter")
            return ss
        import torch.distributed as dist
        if self.size > 1 and a.is_cuda:
            # bf16 partial products, each rank receives only its rows of the sum (NCCL reduce-scatter)
            per = (M + self.size - 1) // self.size
            buf = torch.zeros((self.size * per, N), dtype=a.dtype, device=a.device)
            ops.gemm(a, w, out=buf[:M])
            got = torch.empty((per, N), dtype=a.dtype, device=a.device)
            dist.reduce_scatter_tensor(got, buf, group=self.group)
            mine = (got[:n_own].float() + x_shard[:n_own].float()).to(x_shard.dtype)
        else:
            full = ops.gemm(a, w, out_dtype=torch.float32)
            if self.size > 1:      # gloo has no reduce-scatter
                dist.all_reduce(full, group=self.group)
            mine = (full[lo:lo + n_own] + x_shard[:n_own].float()).to(x_shard.dtype)
        x_shard[:n_own].copy_(mine)
        pad = parts * 256 - N
        sq = mine.float().pow(2)
        if pad:
            sq = torch.nn.functional.pad(sq, (0, pad))
        ss[:n_own].copy_(sq.reshape(n_own, parts, 256).sum(-1))
        return ss

    def allgather_rows(self, a_shard, a_full, ss_out=None):
        """Plain all-gather of row shards into ``a_full`` (no GEMM behind it), with the rows' sums of squares per 256
        columns in ``ss_out`` when given."""
        import torch.distributed as dist
        M, K = a_full.shape
        lo, n_own = self.shard_rows(M)
        if self.size == 1:
            a_full[:n_own].copy_(a_shard[:n_own])
        else:
            per = (M + self.size - 1) // self.size
            buf = torch.zeros((self.size * per, K), dtype=a_full.dtype, device=a_full.device)
            mine = torch.zeros((per, K), dtype=a_full.dtype, device=a_full.device)
            mine[:n_own].copy_(a_shard[:n_own])
            dist.all_gather_into_tensor(buf, mine, group=self.group)
            a_full.copy_(buf[:M])
        if ss_out is not None:
            G = ss_out.shape[1]
            sq = a_full.float().pow(2)
            pad = G * 256 - K
            if pad:
                sq = torch.nn.functional.pad(sq, (0, pad))
            ss_out[:M].copy_(sq.reshape(M, G, 256).sum(-1))
        return a_full

    def allgather_input(self, a_shard, a_full, ss_out=None):
        """Column-parallel GEMM over sequence-parallel activations: the NEXT GEMM op called with ``a_full`` ([M, K]
        local tensor) as its A operand first gathers the ranks' row shards (``a_shard``: this rank's
        ``shard_rows(M)`` rows) into it, inside the same kernel, while its first weight tiles are already in flight.
        Without the fused form the rows are gathered here with an ordinary all-gather. ``ss_out`` [M, K / 256] fp32
        receives the gathered rows' sums of squares per 256 columns (written by the same kernel before its main loop,
        so the GEMM may take it as its ``row_ss``). Reference: tp_column_parallel_all_gather
        (src/engine/coordinator/compute.rs:246-271)."""
        M, K = a_full.shape
        lo, n_own = self.shard_rows(M)
        fused = (self.mode == "fused" and self.form == "ll" and not self.baseline and a_full.is_cuda and
                 M * K * 2 <= self._ag_bytes and K % 256 == 0 and a_full.dtype == torch.bfloat16 and
                 (ss_out is None or (ss_out.is_contiguous() and ss_out.shape[1] == K // 256)))
        if fused:
            rc = nv.lib().gllm_gemm_set_allgather_input(
                a_shard.data_ptr(), a_shard.stride(0), a_full.data_ptr(), a_full.stride(0), self.size, self.rank,
                self._mc_base, ctypes.cast(self._peer_base, ctypes.c_void_p), self._total, self._lay["ag_slots"][0],
                self._ag_bytes, self._ag_state.data_ptr(), nv.ptr(ss_out))
            nv.check(rc, "gemm_set_allgather_input")
            return a_full
        return self.allgather_rows(a_shard, a_full, ss_out)

    def reset(self):
        """Clear the flags, done words and launch state after a failed launch (collective: every rank calls it)."""
        import torch.distributed as dist
        torch.cuda.synchronize(self.device)
        if self.size > 1:
            dist.barrier(group=self.group)
        if self.mode == "fused":
            for name in ("flags", "done", "counters"):
                if name in self._lay:
                    off, nbytes = self._lay[name]
                    self._symm[off:off + nbytes].zero_()
            self._fill_sentinel()
            self._state.zero_()
            self._ag_state.zero_()
        torch.cuda.synchronize(self.device)
        if self.size > 1:
            dist.barrier(group=self.group)

    # ------------------------------------------------------------------------------------------
    def sample_vocab_parallel(self, logits, vocab_local, vocab_start, params, seed, offsets, out, vocab, greedy=True,
                              topk_cap: int = 0):
        """Each rank holds logits for vocabulary rows [vocab_start, vocab_start+vocab_local). Greedy requests
        exchange only (max, argmax) pairs. ``topk_cap`` > 0 (every row samples with 0 < top_k <= topk_cap): each rank
        sends its ``topk_cap`` best (logit, index) pairs per row, the union holds every row's global top-k, and all
        ranks sample from it (top-k first, then top-p inside it, as the sampler orders them): W * topk_cap pairs per row
        on the wire instead of the vocabulary. Otherwise the shards are gathered whole. Every rank samples with the
        same Philox seed and offsets, so all agree on the token without another broadcast."""
        import torch.distributed as dist
        B = logits.shape[0]
        if not greedy and topk_cap > 0:
            k = min(int(topk_cap), int(vocab_local))
            vals, idx = torch.topk(logits[:, :vocab_local].float(), k, dim=1)
            pair = torch.cat([vals, (idx + vocab_start).to(torch.float32)], 1).contiguous()     # indices < 2^24: exact
            allp = torch.empty((self.size * B, 2 * k), dtype=torch.float32, device=logits.device)
            dist.all_gather_into_tensor(allp, pair, group=self.group)
            allp = allp.view(self.size, B, 2 * k)
            cand_vals = allp[:, :, :k].permute(1, 0, 2).reshape(B, self.size * k).contiguous()
            cand_idx = allp[:, :, k:].permute(1, 0, 2).reshape(B, self.size * k)
            pick = ops.sample(cand_vals, params, vocab=self.size * k, seed=seed, step_offsets=offsets)
            out.copy_(cand_idx.gather(1, pick.long()[:, None]).squeeze(1).to(torch.int32))
            return out
        if greedy:
            vals = torch.empty(B, dtype=torch.float32, device=logits.device)
            idx = torch.empty(B, dtype=torch.int32, device=logits.device)
            ops.argmax(logits, vocab_local, out=idx, out_vals=vals)
            pair = torch.stack([vals, (idx + vocab_start).to(torch.float32)], 1).contiguous()
            allp = torch.empty((self.size * B, 2), dtype=torch.float32, device=logits.device)
            dist.all_gather_into_tensor(allp, pair, group=self.group)
            allp = allp.view(self.size, B, 2)
            best = allp[:, :, 0].argmax(0)  # first rank wins ties -> lowest vocabulary index
            out.copy_(allp[best, torch.arange(B, device=logits.device), 1].to(torch.int32))
            return out
        shard = logits[:, :vocab_local].contiguous()
        # shards may differ by one row when vocab % size != 0: pad to the widest
        width = (vocab + self.size - 1) // self.size
        if shard.shape[1] < width:
            shard = torch.nn.functional.pad(shard, (0, width - shard.shape[1]), value=float("-inf"))
        allv = torch.empty((self.size * B, width), dtype=torch.float32, device=logits.device)
        dist.all_gather_into_tensor(allv, shard, group=self.group)
        allv = allv.view(self.size, B, width)
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


def mode_for_comm_config(comm) -> str:
    """``TPContext`` mode for a ``parallel.config.CommConfig``: which of the engine's all-reduce forms stands for each
    algorithm family of the reference's communication layer.

    FLUX_PIPELINE (GEMM fused with its collective) and the automatic choices -> ``auto`` (the low-latency ownership
    form, multimem broadcast when the switch offers it); HARDWARE_REDUCE / COLLNET_DIRECT (in-switch reduction) ->
    ``pull`` (``multimem.ld_reduce``); DIRECT (one-shot peer access) -> ``ll_p2p`` (plain peer stores, no multimem);
    CHUNKED_PIPELINE -> ``fused`` (per-tile pushes with flags); the ring / tree families have no hand-written
    counterpart on an NVSwitch box and take NCCL. ``overlap`` = ``prefer_isolated`` also selects NCCL (collective and
    GEMM as separate kernels). Reference: CommAlgorithm selection (src/engine/coordinator/compute.rs:122-436)."""
    from .config import CommAlgorithm
    if str(getattr(comm, "overlap", "auto")) == "prefer_isolated":
        return "nccl"
    table = {CommAlgorithm.FLUX_PIPELINE: "auto", CommAlgorithm.HARDWARE_REDUCE: "pull", CommAlgorithm.COLLNET_DIRECT: "pull",
             CommAlgorithm.DIRECT: "ll_p2p", CommAlgorithm.CHUNKED_PIPELINE: "fused", CommAlgorithm.RING: "nccl",
             CommAlgorithm.TREE: "nccl", CommAlgorithm.TOPO_AWARE_RING: "nccl", CommAlgorithm.HIERARCHICAL_RING: "nccl"}
    return table.get(getattr(comm, "algorithm", CommAlgorithm.FLUX_PIPELINE), "auto")


def single_gpu_context(device, hidden: int, max_tokens: int = 1024, mode: str = "fused_p2p") -> TPContext:
    """A world-size-1 context on ordinary device memory: exercises the fused kernel's protocol (receive slots, tile
    flags, done words, launch state; with ``mode="ll_p2p"`` the self-validating slots; with ``mode="pull_p2p"``
    alternating buffers and arrival counters) on one GPU."""
    return TPContext(0, 1, device, mode=mode, max_tokens=max_tokens, hidden=hidden)
