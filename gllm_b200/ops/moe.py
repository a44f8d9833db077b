"""Mixture-of-experts ops: routing, permutation into per-expert 128-row blocks, weighted combine.

CUDA path: ``csrc/kernels/moe.cu`` + the grouped tcgen05 GEMM. CPU path / oracle: the reference's scalar
semantics (src/compat/scalar_ops.rs:70-181): softmax over all experts -> top-k -> renormalise.
"""
from __future__ import annotations

import torch

from . import _native as nv
from ._native import F, I, L, P

nv.register("gllm_moe_route", I, [P, L, I, I, I, I, I, P, F, P, P, P])
nv.register("gllm_moe_permute", I, [P, P, I, P, I, I, I, I, I, P, P, P, P, I, P, P, P, P, P])
nv.register("gllm_moe_combine", I, [P, P, P, I, I, I, P, P, P, P])

BLOCK = 128


def route_ref(logits, k, norm_topk=True, scoring="softmax", sel_bias=None, scale=1.0):
    lg = logits.float()
    score = torch.softmax(lg, -1) if scoring == "softmax" else torch.sigmoid(lg)
    sel = score if sel_bias is None else score + sel_bias.float()
    _, ids = torch.topk(sel, k, dim=-1, sorted=True)
    w = torch.gather(score, 1, ids)
    if norm_topk:
        w = w / w.sum(-1, keepdim=True).clamp_min(1e-20)
    return ids.to(torch.int32), w * scale


def route(logits, k, *, norm_topk=True, scoring="softmax", sel_bias=None, scale=1.0, out_ids=None, out_w=None):
    """logits [T,E] fp32 -> (ids [T,k] int32, weights [T,k] fp32)."""
    T, E = logits.shape
    if not logits.is_cuda:
        return route_ref(logits, k, norm_topk, scoring, sel_bias, scale)
    if out_ids is None:
        out_ids = torch.empty((T, k), dtype=torch.int32, device=logits.device)
        out_w = torch.empty((T, k), dtype=torch.float32, device=logits.device)
    rc = nv.lib().gllm_moe_route(logits.data_ptr(), logits.stride(0), T, E, k, 1 if norm_topk else 0,
                                 0 if scoring == "softmax" else 1, nv.ptr(sel_bias), float(scale), out_ids.data_ptr(),
                                 out_w.data_ptr(), nv.stream_ptr())
    nv.check(rc, "moe_route")
    return out_ids, out_w


class MoeWorkspace:
    """Worst-case-sized buffers for one MoE layer invocation (shared by all layers)."""

    def __init__(self, max_tokens, k, hidden, inter, e_local, device, dtype):
        self.max_rows = max_tokens * k + e_local * (BLOCK - 1)
        self.max_rows = (self.max_rows + BLOCK - 1) // BLOCK * BLOCK
        self.max_blocks = self.max_rows // BLOCK
        z = lambda *s, dt=torch.int32: torch.zeros(*s, dtype=dt, device=device)
        self.counts, self.offsets, self.cursors = z(e_local), z(e_local + 1), z(e_local)
        self._blk, self.total_rows = z(2 * self.max_blocks), z(1)
        self.blk_group = self._blk[:self.max_blocks]       # expert of every 128-row block (-1: inactive)
        self.blk_rows = self._blk[self.max_blocks:]        # routed rows in every block (the rest of the block is padding)
        self.a_perm = torch.zeros((self.max_rows, hidden), dtype=dtype, device=device)
        self.ss_perm = torch.ones(self.max_rows, 1, dtype=torch.float32, device=device)
        self.act = torch.zeros((self.max_rows, inter), dtype=dtype, device=device)
        self.y_perm = torch.zeros((self.max_rows, hidden), dtype=dtype, device=device)
        self.dest = z(max_tokens * k)
        self.ids = z(max_tokens, k)
        self.w = torch.zeros((max_tokens, k), dtype=torch.float32, device=device)
        self.logits = None


def permute(x, row_ss, ids, ws: MoeWorkspace, e0=0, e_local=None):
    """Bucket (token, slot) pairs by local expert. Fills ws.a_perm / ss_perm / blk_group / dest."""
    T, k = ids.shape
    H = x.shape[1]
    e_local = e_local if e_local is not None else ws.counts.shape[0]
    if not x.is_cuda:
        flat = ids.reshape(-1).long() - e0
        ok = (flat >= 0) & (flat < e_local)
        counts = torch.bincount(flat[ok], minlength=e_local)
        padded = (counts + BLOCK - 1) // BLOCK * BLOCK
        offs = torch.cat([torch.zeros(1, dtype=torch.long), padded.cumsum(0)])
        ws.offsets.copy_(offs.to(torch.int32))
        ws.total_rows[0] = int(offs[-1])
        ws.dest.fill_(-1)
        cursor = [0] * e_local
        for i in range(T * k):
            if bool(ok[i]):
                e = int(flat[i])
                d = int(offs[e]) + cursor[e]
                cursor[e] += 1
                ws.dest[i] = d
                ws.a_perm[d] = x[i // k]
                if row_ss is not None:
                    ws.ss_perm[d, 0] = row_ss[i // k].float().sum()
        blk = torch.full((ws.max_blocks,), -1, dtype=torch.int32)
        rows = torch.zeros(ws.max_blocks, dtype=torch.int32)
        for b in range(ws.max_blocks):
            r = b * BLOCK
            if r < int(offs[-1]):
                e = int(torch.searchsorted(offs, torch.tensor(r), right=True)) - 1
                blk[b] = e
                rows[b] = min(BLOCK, int(counts[e]) - (r - int(offs[e])))
        ws.blk_group.copy_(blk)
        ws.blk_rows.copy_(rows)
        return
    parts = 0 if row_ss is None else (row_ss.shape[1] if row_ss.dim() > 1 else 1)
    rc = nv.lib().gllm_moe_permute(x.data_ptr(), nv.ptr(row_ss), parts, ids.data_ptr(), T, k, H, e0, e_local,
                                   ws.counts.data_ptr(), ws.offsets.data_ptr(), ws.cursors.data_ptr(),
                                   ws.blk_group.data_ptr(), ws.max_blocks, ws.total_rows.data_ptr(),
                                   ws.a_perm.data_ptr(), ws.ss_perm.data_ptr() if row_ss is not None else None,
                                   ws.dest.data_ptr(), nv.stream_ptr())
    nv.check(rc, "moe_permute")


def combine(x, y_perm, dest, weights, *, shared=None, ss_out=None):
    """x[t] += sum_k w[t,k] * y_perm[dest[t,k]] (+ shared[t]); in place; ss_out[t] = sum(x[t]^2)."""
    T, k = weights.shape
    H = x.shape[1]
    if not x.is_cuda:
        d = dest[:T * k].reshape(T, k).long()
        ok = d >= 0
        rows = y_perm[d.clamp_min(0)].float() * (weights.float() * ok)[..., None]
        acc = x.float() + rows.sum(1)
        if shared is not None:
            acc = acc + shared.float()
        x.copy_(acc.to(x.dtype))
        if ss_out is not None:
            ss_out.reshape(-1)[:T].copy_(x.float().pow(2).sum(-1))
        return x
    rc = nv.lib().gllm_moe_combine(y_perm.data_ptr(), dest.data_ptr(), weights.data_ptr(), T, k, H, nv.ptr(shared),
                                   x.data_ptr(), nv.ptr(ss_out), nv.stream_ptr())
    nv.check(rc, "moe_combine")
    return x
