"""Expert parallelism: every rank owns ``E / ep`` consecutive experts and its own tokens (data-parallel
attention); routed hidden rows travel to the expert's rank and the expert outputs travel back.

Two transports:

* ``fused`` (CUDA, NVLink peers): ``csrc/kernels/ep.cu``. The dispatch kernel writes each routed row straight
  into the owning rank's grouped-GEMM input buffer with peer stores; the second expert GEMM scatters its output
  rows into the token owner's memory as its tiles retire (``gllm_gemm_bf16_grouped_scatter``); the combine kernel
  then reads only local memory. Four flag waits per layer, no host synchronisation, CUDA-graph replayable.
* ``a2a`` (NCCL / gloo): three ``all_to_all_single`` calls with a host read of the split sizes. It is the
  baseline the fused transport is measured against and the path the CPU multi-process tests exercise.

Reference parity: ``dispatch_experts`` + ``all_to_all_exchange_counts`` (src/moe/distributed_dispatch.rs:160-284)
group token indices by target rank and all-gather the counts; the token exchange itself was never implemented
there. Placement is the contiguous one (``MoePlacement.AUTO``).
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from ..ops import _native as nv
from ..ops import linear as L
from ..ops import moe as M
from ..ops._native import I, L as LL, P

nv.register("gllm_ep_dispatch", I, [P, P, P, I, P, I, I, P, P, I, P, P])
nv.register("gllm_ep_combine", I, [P, P, P, I, I, P, P, P, P])
nv.register("gllm_gemm_bf16_grouped_scatter", I, [P, LL, P, LL, LL, I, I, I, P, I, I, P, P, I, P, I])

BLOCK = 128


class _EpDesc(ctypes.Structure):
    _fields_ = [("world", ctypes.c_int), ("rank", ctypes.c_int), ("num_experts", ctypes.c_int),
                ("e_local", ctypes.c_int), ("hidden", ctypes.c_int), ("max_rows", ctypes.c_int),
                ("counts", ctypes.c_void_p * 8), ("flags", ctypes.c_void_p * 8), ("x", ctypes.c_void_p * 8),
                ("ss", ctypes.c_void_p * 8), ("meta", ctypes.c_void_p * 8), ("state", ctypes.c_void_p),
                ("cta_done", ctypes.c_void_p)]


def _align(n, a=256):
    return (n + a - 1) // a * a


class EPContext:
    def __init__(self, rank: int, size: int, device, *, num_experts: int, hidden: int, top_k: int,
                 max_tokens: int = 256, mode: str = "auto", group=None, dtype=torch.bfloat16):
        if num_experts % size:
            raise ValueError(f"num_experts ({num_experts}) must be divisible by the expert-parallel size ({size})")
        self.rank, self.size, self.device = rank, size, torch.device(device)
        self.group, self.dtype = group, dtype
        self.num_experts, self.e_local, self.hidden, self.top_k = num_experts, num_experts // size, hidden, top_k
        self.max_tokens = max_tokens
        self.token_bound = max_tokens       # callers may lower it per step (all ranks alike) to bound GEMM grids
        self.max_rows = _align(size * max_tokens * top_k + self.e_local * (BLOCK - 1), BLOCK)
        self.max_blocks = self.max_rows // BLOCK
        self.mode = "a2a"
        self._act = {}
        self._a2a_ws = {}
        if mode in ("auto", "fused") and self.device.type == "cuda":
            try:
                self._setup_fused()
                self.mode = "fused"
            except Exception as exc:
                if mode == "fused":
                    raise
                self.setup_error = repr(exc)

    # ------------------------------------------------------------------------------------------
    def _setup_fused(self):
        E, H, k = self.num_experts, self.hidden, self.top_k
        if H % 128:
            raise ValueError("the fused expert-parallel transport needs hidden % 128 == 0")
        sizes = [("counts", self.size * E * 4), ("flags", 64), ("x", self.max_rows * H * 2), ("ss", self.max_rows * 4),
                 ("meta", self.max_rows * 4), ("y", self.max_tokens * k * H * 2)]
        offs, total = {}, 0
        for name, nbytes in sizes:
            offs[name] = total
            total += _align(nbytes)
        if self.size == 1:
            buf = torch.zeros(total, dtype=torch.uint8, device=self.device)
            peers = [buf.data_ptr()]
        else:
            import torch.distributed as dist
            import torch.distributed._symmetric_memory as symm_mem
            group = self.group or dist.group.WORLD
            buf = symm_mem.empty(total, dtype=torch.uint8, device=self.device)
            self._handle = symm_mem.rendezvous(buf, group.group_name)
            buf.zero_()
            torch.cuda.synchronize(self.device)
            dist.barrier(group=group)
            peers = [int(p) for p in self._handle.buffer_ptrs]
        self._buf, self._offs = buf, offs
        view = lambda name, dt, shape: buf[offs[name]: offs[name] + _align(dict(sizes)[name])].view(dt)[
            : int(torch.tensor(shape).prod())].view(*shape)
        self.x_recv = view("x", torch.bfloat16, (self.max_rows, H))
        self.ss_recv = view("ss", torch.float32, (self.max_rows, 1))
        self.meta = view("meta", torch.int32, (self.max_rows,))
        self.y_gather = view("y", torch.bfloat16, (self.max_tokens * k, H))
        self.meta.fill_(-1)
        self.ss_recv.fill_(1.0)
        z = lambda n, dt=torch.int32: torch.zeros(n, dtype=dt, device=self.device)
        self.state, self.cta_done, self.cursors = z(1, torch.int64), z(1), z(E)
        self._blk = torch.full((2 * self.max_blocks,), -1, dtype=torch.int32, device=self.device)
        self.blk_group, self.blk_rows = self._blk[:self.max_blocks], self._blk[self.max_blocks:]   # expert / received rows per block
        self.total_rows = z(1)
        d = _EpDesc()
        d.world, d.rank, d.num_experts, d.e_local, d.hidden, d.max_rows = self.size, self.rank, E, self.e_local, H, self.max_rows
        for r, base in enumerate(peers):
            d.counts[r], d.flags[r], d.x[r] = base + offs["counts"], base + offs["flags"], base + offs["x"]
            d.ss[r], d.meta[r] = base + offs["ss"], base + offs["meta"]
        d.state, d.cta_done = self.state.data_ptr(), self.cta_done.data_ptr()
        self._desc = d
        self._y_peers = (ctypes.c_void_p * 8)(*([p + offs["y"] for p in peers] + [None] * (8 - len(peers))))
        if self.size > 1:
            torch.cuda.synchronize(self.device)
            import torch.distributed as dist
            dist.barrier(group=self.group or dist.group.WORLD)

    def rows_bound(self) -> int:
        """Rows the grouped GEMMs have to look at this step (inactive blocks beyond the plan are skipped anyway)."""
        b = _align(self.size * min(self.token_bound, self.max_tokens) * self.top_k + self.e_local * (BLOCK - 1), BLOCK)
        return min(b, self.max_rows)

    def act_buffer(self, inter: int):
        a = self._act.get(inter)
        if a is None:
            a = self._act[inter] = torch.zeros((self.max_rows, inter), dtype=self.dtype, device=self.device)
        return a

    # ------------------------------------------------------------------------------------------
    def dispatch(self, x, row_ss, ids, T):
        parts = 0 if row_ss is None else (row_ss.shape[1] if row_ss.dim() > 1 else 1)
        rc = nv.lib().gllm_ep_dispatch(ctypes.byref(self._desc), x.data_ptr(), nv.ptr(row_ss), parts, ids.data_ptr(),
                                       T, ids.shape[1], self.cursors.data_ptr(), self.blk_group.data_ptr(),
                                       self.max_blocks, self.total_rows.data_ptr(), nv.stream_ptr())
        nv.check(rc, "ep_dispatch")

    def grouped_scatter(self, act, w_down, rows):
        N, K = w_down.shape[0] // self.e_local, w_down.shape[1]
        L.set_block_rows(self.blk_rows)
        rc = nv.lib().gllm_gemm_bf16_grouped_scatter(
            act.data_ptr(), act.stride(0), w_down.data_ptr(), w_down.stride(0), self.hidden, rows, N, K,
            self.blk_group.data_ptr(), self.e_local, 128, self.meta.data_ptr(),
            ctypes.cast(self._y_peers, ctypes.c_void_p), self.size, nv.stream_ptr(), 0)
        nv.check(rc, "gemm_grouped_scatter")

    def combine(self, x, w, T, shared, ss_out):
        rc = nv.lib().gllm_ep_combine(ctypes.byref(self._desc), self.y_gather.data_ptr(), w.data_ptr(), T, w.shape[1],
                                      nv.ptr(shared), x.data_ptr(), nv.ptr(ss_out), nv.stream_ptr())
        nv.check(rc, "ep_combine")

    # ------------------------------------------------------------------------------------------
    def moe_forward(self, layer, model, x, ss_in, ss_out, ids, w, ws, T, *, normalised_input=None):
        """Routed-expert part of one MoE layer for this rank's T tokens. ``x`` [T, H] is updated in place
        (residual add). With ``normalised_input`` (unfused models) that tensor is dispatched instead of ``x``."""
        c = layer.cfg
        H = c.hidden_size
        src = x if normalised_input is None else normalised_input
        fused_norm = normalised_input is None and ss_in is not None
        shared = None
        ss = None if ss_out is None else ss_out.reshape(-1)[:T].view(T, 1)
        if self.mode != "fused":
            return self._forward_a2a(layer, model, x, src, ss_in if fused_norm else None, ss, ids, w, T)
        if T > self.max_tokens:
            raise ValueError(f"{T} tokens exceed the expert-parallel buffers ({self.max_tokens})")
        self.dispatch(src, ss_in if fused_norm else None, ids, T)
        rows = self.rows_bound()
        act = self.act_buffer(layer.inter)
        if getattr(layer, "bs_fmt", None) is None:
            L.set_block_rows(self.blk_rows)
            L.gemm_glu(self.x_recv[:rows], layer.w_gate_up, act=model.act_id, out=act[:rows],
                       row_ss=self.ss_recv[:rows] if fused_norm else None, norm_dim=H if fused_norm else 0,
                       eps=c.rms_norm_eps if fused_norm else 0.0, bn=layer.glu_bn, mblk_group=self.blk_group,
                       num_groups=self.e_local)
            self.grouped_scatter(act, layer.w_down, rows)
        else:
            self._bs_experts(layer, model, act, rows, fused_norm, H)
        if layer.shared_gate_up is not None:
            shared = self._shared(layer, model, src, ss_in if fused_norm else None, H)
        self.combine(x, w, T, shared, ss)
        return ss

    def _bs_experts(self, layer, model, act, rows, fused_norm, H):
        """Block-scaled experts: the received rows (bf16, as the peers stored them) are quantised in place of the bf16
        A operand, only as many as arrived (a count on the device); the SwiGLU output likewise; the second GEMM's
        epilogue scatters its rows back to their source ranks as the bf16 path does."""
        from ..ops import blockscale as B
        c = layer.cfg
        fmt = layer.bs_fmt
        key = (fmt, layer.inter)
        q = self._bsq.get(key) if hasattr(self, "_bsq") else None
        if q is None:
            if not hasattr(self, "_bsq"):
                self._bsq = {}
            q = self._bsq[key] = (B.alloc_act(self.max_rows, H, fmt, self.device),
                                  B.alloc_act(self.max_rows, layer.inter, fmt, self.device))
        xq, aq = q
        ts = layer.act_tensor_scale
        B.quantize_act_rows(self.x_recv, fmt, xq, self.total_rows, tensor_scale=ts)
        xq.rows = rows
        rs = dict(row_ss=self.ss_recv[:rows], norm_dim=H, eps=c.rms_norm_eps) if fused_norm else {}
        L.set_block_rows(self.blk_rows)
        B.gemm_glu(xq, layer.w_gate_up, act=model.act_id, out=act[:rows], bn=128, mblk_group=self.blk_group,
                   num_groups=self.e_local, **rs)
        B.quantize_act_rows(act, fmt, aq, self.total_rows, tensor_scale=ts)
        aq.rows = rows
        L.set_block_rows(self.blk_rows)
        B.gemm_grouped_scatter(aq, layer.w_down, self.blk_group, self.e_local, ldo=self.hidden, scatter_meta=self.meta,
                               scatter_peers=self._y_peers, world=self.size)

    @staticmethod
    def _shared(layer, model, src, ss_in, H):
        from .. import ops
        c = layer.cfg
        sa = L.gemm_glu(src, layer.shared_gate_up, act=model.act_id, row_ss=ss_in, norm_dim=H if ss_in is not None else 0,
                        eps=c.rms_norm_eps if ss_in is not None else 0.0, bn=layer.shared_bn)
        return ops.gemm(sa, layer.shared_down, out_dtype=src.dtype, bn=128)

    # ------------------------------------------------------------------------------------------
    def _forward_a2a(self, layer, model, x, src, ss_in, ss, ids, w, T):
        import torch.distributed as dist
        c = layer.cfg
        H, k = c.hidden_size, ids.shape[1]
        dev = x.device
        flat = ids.reshape(-1).long()
        owner = flat // self.e_local
        order = torch.argsort(owner, stable=True)
        send_counts = torch.bincount(owner, minlength=self.size)
        recv_counts = torch.empty_like(send_counts)
        if self.size > 1:
            dist.all_to_all_single(recv_counts, send_counts, group=self.group)
        else:
            recv_counts.copy_(send_counts)
        sc, rcv = send_counts.tolist(), recv_counts.tolist()
        n = sum(rcv)
        rows = src.index_select(0, order // k).contiguous()
        eids = flat[order].to(torch.int32).contiguous()
        recv_rows = torch.empty((n, H), dtype=src.dtype, device=dev)
        recv_e = torch.empty(n, dtype=torch.int32, device=dev)
        recv_ss = None
        if self.size > 1:
            dist.all_to_all_single(recv_rows, rows, rcv, sc, group=self.group)
            dist.all_to_all_single(recv_e, eids, rcv, sc, group=self.group)
        else:
            recv_rows, recv_e = rows, eids
        if ss_in is not None:
            tok_ss = (ss_in.float().sum(-1) if ss_in.dim() > 1 else ss_in.float()).index_select(0, order // k).contiguous()
            recv_ss = torch.empty(n, dtype=torch.float32, device=dev)
            if self.size > 1:
                dist.all_to_all_single(recv_ss, tok_ss, rcv, sc, group=self.group)
            else:
                recv_ss = tok_ss
        y_rows = torch.zeros((n, H), dtype=src.dtype, device=dev)
        if n > 0:
            key = (max(256, 1 << (n - 1).bit_length()), layer.inter)
            ws2 = self._a2a_ws.get(key)
            if ws2 is None:
                ws2 = self._a2a_ws[key] = M.MoeWorkspace(key[0], 1, H, layer.inter, self.e_local, dev, src.dtype)
            M.permute(recv_rows, None if recv_ss is None else recv_ss.view(n, 1), recv_e.view(n, 1), ws2,
                      self.rank * self.e_local, self.e_local)
            fused_norm = recv_ss is not None
            L.gemm_glu(ws2.a_perm, layer.w_gate_up, act=model.act_id, out=ws2.act,
                       row_ss=ws2.ss_perm if fused_norm else None, norm_dim=H if fused_norm else 0,
                       eps=c.rms_norm_eps if fused_norm else 0.0, bn=layer.glu_bn, mblk_group=ws2.blk_group,
                       num_groups=self.e_local)
            L.gemm_grouped(ws2.act, layer.w_down, ws2.blk_group, self.e_local, out=ws2.y_perm, bn=128)
            y_rows = ws2.y_perm.index_select(0, ws2.dest[:n].long())
        back = torch.empty((T * k, H), dtype=src.dtype, device=dev)
        if self.size > 1:
            dist.all_to_all_single(back, y_rows.contiguous(), sc, rcv, group=self.group)
        else:
            back = y_rows
        y_gather = torch.empty_like(back)
        y_gather[order] = back
        shared = None
        if layer.shared_gate_up is not None:
            shared = self._shared(layer, model, src, ss_in, H)
        dest = torch.arange(T * k, dtype=torch.int32, device=dev)
        M.combine(x, y_gather, dest, w, shared=shared, ss_out=ss)
        return ss

    def close(self):
        self._buf = None
        self._handle = None
