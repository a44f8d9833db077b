"""Mixture-of-experts FFN block (Qwen3-MoE / Mixtral / DeepSeek-style) for the decoder.

Per token: router -> top-k -> the k experts' SwiGLU FFNs -> weighted sum (+ shared expert), added to the
residual stream. Expert weights are stacked ``[E_local * 2I, H]`` (tile-interleaved gate/up) and
``[E_local * H, I]`` so one grouped tcgen05 GEMM serves every routed row; with expert parallelism each rank
holds ``E / ep`` experts and ``parallel/expert_parallel.py`` moves the rows.

Reference parity: MoEGate -> TopK -> masked per-expert template -> MoEConditionalAdd + shared expert
(src/arch/auto_graph_fragments/build_graph.inc.rs:2046-2178), scalar semantics
(src/compat/scalar_ops.rs:70-181).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from .. import ops
from ..ops import linear as L
from ..ops import moe as M
from .config import ModelConfig
from .weights import _fold, layer_prefix, shard_range


@dataclass
class MoeLayerWeights:
    router: torch.Tensor                 # [E, H] (post-attention norm folded in when fused)
    router_bias: Optional[torch.Tensor]  # selection bias (DeepSeek) fp32 [E]
    w_gate_up: torch.Tensor              # [E_local * 2I, H], per expert tile-interleaved
    w_down: torch.Tensor                 # [E_local * H, I]
    glu_bn: int
    e0: int
    e_local: int
    inter: int
    shared_gate_up: Optional[torch.Tensor] = None
    shared_down: Optional[torch.Tensor] = None
    shared_bn: int = 128
    cfg: Optional[ModelConfig] = None
    fused: bool = True
    ep: Optional[object] = None
    tp_experts: Optional[object] = None  # tensor-parallel context when the experts are split over the TP ranks
    bs_fmt: Optional[str] = None         # "mxfp8" / "nvfp4": the expert stacks are block-scaled operands (ops/blockscale.py)
    act_tensor_scale: float = 1.0 / 64.0
    _ws: Optional[M.MoeWorkspace] = None
    paged: Optional["PagedExperts"] = None   # expert stacks in host memory, a few slots of them on the device
    # hot experts mirrored on every rank of the expert-sharded tensor-parallel mode (set_mirrors): their stacks sit
    # behind the rank's own experts, mirror_map[e] is the mirror slot of expert e (-1: not mirrored)
    n_mirror: int = 0
    mirror_map: Optional[torch.Tensor] = None
    mirrored: tuple = ()

    # ------------------------------------------------------------------------------------------
    def workspace(self, model, T):
        holder = model.__dict__.setdefault("_moe_ws", {})
        groups = self.paged.slots if self.paged is not None else self.e_local + self.n_mirror   # paged experts: slots
        key = (groups, self.inter)
        ws = holder.get(key)
        if ws is None or ws.ids.shape[0] < T:
            c = self.cfg
            ws = M.MoeWorkspace(max(T, 256), c.num_experts_per_tok, c.hidden_size, self.inter, groups,
                                model.device, model.dtype)
            ws.logits = torch.zeros((max(T, 256), self.router.shape[0]), dtype=torch.float32, device=model.device)
            holder[key] = ws
        return ws

    def _expert_ffn(self, model, src, ws, T, fused_norm: bool, mark=lambda name: None):
        """The routed rows through their experts' SwiGLU FFNs: ws.y_perm <- down(glu(gate/up(rows))). ``src`` [T, H]
        is what the experts read; the rows were bucketed by ``M.permute`` (ws.dest / blk_group / ss_perm)."""
        c = self.cfg
        H = c.hidden_size
        rs = dict(row_ss=ws.ss_perm, norm_dim=H, eps=c.rms_norm_eps) if fused_norm else {}
        if self.bs_fmt is None:
            # paged experts: the stacks are the device slots, the "experts" of the block table are slot numbers
            w_gu, w_dn, groups = (self.paged.dev_gu, self.paged.dev_dn, self.paged.slots) if self.paged is not None else (
                self.w_gate_up, self.w_down, self.e_local + self.n_mirror)
            rows = getattr(ws, "blk_rows", None)      # routed rows per block: padding rows are neither loaded nor stored
            L.set_block_rows(rows)
            L.gemm_glu(ws.a_perm, w_gu, act=model.act_id, out=ws.act, bn=self.glu_bn, mblk_group=ws.blk_group,
                       num_groups=groups, **rs)
            mark("moe_gate_up")
            L.set_block_rows(rows)
            L.gemm_grouped(ws.act, w_dn, ws.blk_group, groups, out=ws.y_perm, bn=128)
            mark("moe_down")
            return
        # block-scaled experts: the routed rows are quantised straight from the token rows into their expert blocks,
        # the SwiGLU output is quantised again for the down projection (only the rows that exist: a device-side count)
        from ..ops import blockscale as B
        k = c.num_experts_per_tok
        if getattr(ws, "aq", None) is None or ws.aq.fmt != B.FMT_NAMES[self.bs_fmt]:
            ws.aq = B.alloc_act(ws.max_rows, H, self.bs_fmt, src.device)
            ws.actq = B.alloc_act(ws.max_rows, self.inter, self.bs_fmt, src.device)
        ts = self.act_tensor_scale
        B.quantize_act_scatter(src, ws.dest, k, self.bs_fmt, ws.aq, ws.max_rows, tensor_scale=ts)
        mark("moe_quant_in")
        rows = getattr(ws, "blk_rows", None)
        L.set_block_rows(rows)
        B.gemm_glu(ws.aq, self.w_gate_up, act=model.act_id, out=ws.act, bn=128, mblk_group=ws.blk_group,
                   num_groups=self.e_local, **rs)
        mark("moe_gate_up")
        B.quantize_act_rows(ws.act, self.bs_fmt, ws.actq, ws.total_rows, tensor_scale=ts)
        mark("moe_quant_mid")
        L.set_block_rows(rows)
        B.gemm(ws.actq, self.w_down, out=ws.y_perm, bn=128, mblk_group=ws.blk_group, num_groups=self.e_local)
        mark("moe_down")

    def _route(self, x, row_ss, ws, T, norm_dim, eps):
        c = self.cfg
        logits = ops.gemm(x, self.router, out=ws.logits[:T], out_dtype=torch.float32, row_ss=row_ss,
                          norm_dim=norm_dim, eps=eps, bn=128)
        E = c.num_experts
        ids, w = M.route(logits[:, :E], c.num_experts_per_tok, norm_topk=c.norm_topk_prob, scoring=c.router_scoring,
                         sel_bias=self.router_bias, scale=c.routed_scaling_factor,
                         out_ids=ws.ids[:T] if x.is_cuda else None, out_w=ws.w[:T] if x.is_cuda else None)
        ws.last_ids = ids      # the load balancer samples the most recent routing decision from here
        return ids, w

    def forward(self, model, x, ss_in, ss_out, T):
        """Fused path: ``x`` is the residual stream (bf16), ``ss_in`` its row statistics; the post-attention
        RMSNorm is folded into the router and gate/up weights. Returns the statistics tensor of the new x."""
        c = self.cfg
        H = c.hidden_size
        ws = self.workspace(model, T)
        tm = getattr(model, "op_timer", None)      # per-op device time inside a CUDA graph (bench --op-breakdown)
        mark = tm.mark if tm is not None else (lambda name: None)
        ids, w = self._route(x, ss_in, ws, T, H, c.rms_norm_eps)
        mark("moe_route")
        if self.ep is not None:
            return self.ep.moe_forward(self, model, x, ss_in, ss_out, ids, w, ws, T)
        if self.tp_experts is not None:
            return self._forward_tp_experts(model, x, x, ss_in, ss_out, ids, w, ws, T, fused_norm=True)
        if self.paged is not None:
            return self._forward_paged(model, x, x, ss_in, ss_out, ids, w, ws, T, fused_norm=True)
        M.permute(x, ss_in, ids, ws, self.e0, self.e_local)
        mark("moe_permute")
        self._expert_ffn(model, x, ws, T, fused_norm=True, mark=mark)
        shared = None
        if self.shared_gate_up is not None:
            sa = L.gemm_glu(x, self.shared_gate_up, act=model.act_id, row_ss=ss_in, norm_dim=H, eps=c.rms_norm_eps,
                            bn=self.shared_bn)
            shared = ops.gemm(sa, self.shared_down, bn=128)
        ss = ss_out.reshape(-1)[:T].view(T, 1)
        M.combine(x, ws.y_perm, ws.dest, w, shared=shared, ss_out=ss)
        mark("moe_combine")
        return ss

    def _forward_tp_experts(self, model, x, src, ss_in, ss_out, ids, w, ws, T, fused_norm: bool):
        """Tensor-parallel attention + expert-parallel FFN on the same ranks: the tokens are replicated, so each
        rank runs only ITS experts on the rows routed to them and the weighted partial sums are all-reduced
        (same bytes on the wire as dispatch + combine, no token exchange). ``src`` is what the experts read
        (the residual stream with the norm folded into the weights, or the normalised hidden)."""
        import torch.distributed as dist
        c = self.cfg
        H = c.hidden_size
        if self.n_mirror:
            # rows routed to a mirrored (hot) expert are shared out over the ranks by token index; every other row
            # stays with the rank that owns its expert
            tpc = self.tp_experts
            m = self.mirror_map.index_select(0, ids.reshape(-1).long()).reshape(ids.shape)          # -1 or mirror slot
            mine = (torch.arange(T, device=ids.device)[:, None] % tpc.size) == tpc.rank
            out_of_range = torch.full_like(ids, c.num_experts + self.n_mirror + 1)
            own = (ids >= self.e0) & (ids < self.e0 + self.e_local)       # the mirror slots extend the local id range:
            ids_local = torch.where(m >= 0, torch.where(mine, (self.e0 + self.e_local + m).to(ids.dtype), out_of_range),
                                    torch.where(own, ids, out_of_range))     # other ranks' experts must stay outside it
            M.permute(src, ss_in if fused_norm else None, ids_local.contiguous(), ws, self.e0, self.e_local + self.n_mirror)
        else:
            M.permute(src, ss_in if fused_norm else None, ids, ws, self.e0, self.e_local)
        self._expert_ffn(model, src, ws, T, fused_norm)
        holder = model.__dict__.setdefault("_moe_partial", {})
        part = holder.get("buf")
        if part is None or part.shape[0] < T:
            part = holder["buf"] = torch.zeros((max(T, 256), H), dtype=x.dtype, device=x.device)
        p = part[:T]
        p.zero_()
        M.combine(p, ws.y_perm, ws.dest, w)            # this rank's share of sum_k w_k * expert_k(x)
        tp = self.tp_experts
        if tp.size > 1:
            dist.all_reduce(p, group=tp.group)
        if self.shared_gate_up is not None:               # replicated: added once, after the reduction
            sa = L.gemm_glu(src, self.shared_gate_up, act=model.act_id, row_ss=ss_in if fused_norm else None,
                            norm_dim=H if fused_norm else 0, eps=c.rms_norm_eps if fused_norm else 0.0, bn=self.shared_bn)
            p.add_(ops.gemm(sa, self.shared_down, out_dtype=x.dtype, bn=128))
        ss = None if ss_out is None else ss_out.reshape(-1)[:T].view(T, 1)
        ops.rmsnorm(p, None, 0.0, residual=x, h_out=x, ss_out=ss, want_y=False)
        return ss

    def set_mirrors(self, hot, model=None):
        """Load-balancer placement for the expert-sharded tensor-parallel mode: the ``hot`` experts are mirrored on
        every rank (their weights are broadcast from the owner and stacked behind the rank's own experts) and their
        rows are shared out over the ranks; ``hot = []`` goes back to the plain placement. A collective: every rank of
        the tensor-parallel group calls it with the same list. Reference: HotCold placement with mirrored hot experts
        (src/moe/distributed_dispatch.rs:19-285, src/moe/eplb.rs:180-243)."""
        import torch.distributed as dist
        tpc = self.tp_experts
        if tpc is None or self.bs_fmt is not None or self.paged is not None:
            raise ValueError("mirrors: bf16 experts sharded over the tensor-parallel ranks only")
        hot = sorted(set(int(e) for e in hot))
        rows_gu = self.w_gate_up.shape[0] // (self.e_local + self.n_mirror)
        rows_dn = self.w_down.shape[0] // (self.e_local + self.n_mirror)
        own_gu, own_dn = self.w_gate_up[:self.e_local * rows_gu], self.w_down[:self.e_local * rows_dn]
        per = self.cfg.num_experts // tpc.size
        gus, dns = [own_gu], [own_dn]
        for e in hot:
            owner = e // per
            g = torch.empty((rows_gu, own_gu.shape[1]), dtype=own_gu.dtype, device=own_gu.device)
            d = torch.empty((rows_dn, own_dn.shape[1]), dtype=own_dn.dtype, device=own_dn.device)
            if tpc.rank == owner:
                l = e - self.e0
                g.copy_(own_gu[l * rows_gu:(l + 1) * rows_gu])
                d.copy_(own_dn[l * rows_dn:(l + 1) * rows_dn])
            if tpc.size > 1:
                src_rank = dist.get_global_rank(tpc.group, owner) if tpc.group is not None else owner
                dist.broadcast(g, src=src_rank, group=tpc.group)
                dist.broadcast(d, src=src_rank, group=tpc.group)
            gus.append(g)
            dns.append(d)
        self.w_gate_up, self.w_down = torch.cat(gus, 0).contiguous(), torch.cat(dns, 0).contiguous()
        self.n_mirror, self.mirrored = len(hot), tuple(hot)
        mm = torch.full((self.cfg.num_experts,), -1, dtype=torch.int32, device=own_gu.device)
        for slot, e in enumerate(hot):
            mm[e] = slot
        self.mirror_map = mm
        if model is not None:
            model.__dict__.get("_moe_ws", {}).clear()      # the block tables have one more group per mirror

    def _forward_paged(self, model, x, src, ss_in, ss_out, ids, w, ws, T, fused_norm: bool):
        """Experts paged in from host memory: the step's experts are made resident wave by wave (as many as there are
        device slots), each wave runs the ordinary grouped GEMMs over the slots and adds its weighted rows to a
        partial sum; the residual add (and the next norm's statistics) follow once. Costs one host read of the routing
        per layer, the price of serving a model whose experts do not fit the device."""
        c = self.cfg
        H = c.hidden_size
        pg = self.paged
        holder = model.__dict__.setdefault("_moe_partial", {})
        part = holder.get("buf")
        if part is None or part.shape[0] < T:
            part = holder["buf"] = torch.zeros((max(T, 256), H), dtype=x.dtype, device=x.device)
        p = part[:T]
        p.zero_()
        # where each of the step's experts runs: resident ones on the device right away, with host compute enabled a
        # bounded share of the rows (experts with few rows that are not resident) on the host from the host copy of the
        # weights, the rest is fetched (moe.routing.MoeHardwareDispatcher: gpu / cpu / remote)
        from ..moe.routing import MoeHardwareDispatcher
        flat = ids.reshape(-1).long() - self.e0
        local = flat[(flat >= 0) & (flat < self.e_local)]
        counts = torch.bincount(local, minlength=self.e_local).tolist()
        pg.thermal.step(counts)
        plan = MoeHardwareDispatcher(list(pg.slot_of), max_cpu_ratio=pg.max_cpu_ratio,
                                     cpu_enabled=pg.cpu_experts).dispatch(counts)
        pg.last_plan = plan
        used = [a.expert_idx for a in plan.gpu_experts] + [a.expert_idx for a in plan.remote_experts]
        pg.after_gate(ids)
        for a in plan.cpu_experts:
            pg.run_on_host(a.expert_idx, src, ss_in if fused_norm else None, ids, w, p, self, model)
        for i in range(0, len(used), pg.slots):
            wave = used[i:i + pg.slots]
            pg.ensure(wave)
            slot_ids = pg.slot_map(wave).index_select(0, (ids.reshape(-1).long() - self.e0).clamp_(0, self.e_local - 1))
            outside = (ids.reshape(-1) < self.e0) | (ids.reshape(-1) >= self.e0 + self.e_local)
            slot_ids = torch.where(outside, torch.full_like(slot_ids, pg.slots), slot_ids).reshape(ids.shape).contiguous()
            M.permute(src, ss_in if fused_norm else None, slot_ids, ws, 0, pg.slots)
            self._expert_ffn(model, src, ws, T, fused_norm)
            M.combine(p, ws.y_perm, ws.dest, w)
        if self.shared_gate_up is not None:
            sa = L.gemm_glu(src, self.shared_gate_up, act=model.act_id, row_ss=ss_in if fused_norm else None,
                            norm_dim=H if fused_norm else 0, eps=c.rms_norm_eps if fused_norm else 0.0, bn=self.shared_bn)
            p.add_(ops.gemm(sa, self.shared_down, out_dtype=x.dtype, bn=128))
        ss = None if ss_out is None else ss_out.reshape(-1)[:T].view(T, 1)
        ops.rmsnorm(p, None, 0.0, residual=x, h_out=x, ss_out=ss, want_y=False)
        return ss

    def forward_unfused(self, model, x, h, T):
        """Unfused path: ``h`` is the already normalised input; adds the MoE output into ``x``."""
        c = self.cfg
        ws = self.workspace(model, T)
        ids, w = self._route(h, None, ws, T, 0, 0.0)
        if self.ep is not None:
            self.ep.moe_forward(self, model, x, None, None, ids, w, ws, T, normalised_input=h)
            return
        if self.tp_experts is not None:
            self._forward_tp_experts(model, x, h, None, None, ids, w, ws, T, fused_norm=False)
            return
        if self.paged is not None:
            self._forward_paged(model, x, h, None, None, ids, w, ws, T, fused_norm=False)
            return
        M.permute(h, None, ids, ws, self.e0, self.e_local)
        self._expert_ffn(model, h, ws, T, fused_norm=False)
        shared = None
        if self.shared_gate_up is not None:
            sa = L.gemm_glu(h, self.shared_gate_up, act=model.act_id, bn=self.shared_bn)
            shared = ops.gemm(sa, self.shared_down, out_dtype=x.dtype, bn=128)
        M.combine(x, ws.y_perm, ws.dest, w, shared=shared)


def pack_moe_layer(cfg: ModelConfig, src, i: int, tp_rank: int, tp_size: int, device, dtype, ep=None, fused=True, tp=None,
                   expert_quant: Optional[str] = None):
    """Experts are split over the expert-parallel group (``ep``), or kept whole when there is none; the shared
    expert and the router are replicated."""
    p = layer_prefix(i)
    ep_rank, ep_size = (ep.rank, ep.size) if ep is not None else (0, 1)
    tp_experts = None
    if ep is None and tp is not None and tp_size > 1 and cfg.num_experts % tp_size == 0 and getattr(tp, "shard_experts", True):
        # tensor-parallel attention + expert-parallel FFN on the same ranks
        ep_rank, ep_size, tp_experts = tp_rank, tp_size, tp
    e0, e1 = shard_range(cfg.num_experts, ep_rank, ep_size)
    post = src.get(p + "post_attn_norm").float().to(device)
    inter = cfg.moe_intermediate_size
    bn = 256 if inter % 128 == 0 else 128
    gus, downs = [], []
    for e in range(e0, e1):
        g = src.get(f"{p}experts.{e}.gate_proj").to(device, dtype)
        u = src.get(f"{p}experts.{e}.up_proj").to(device, dtype)
        d = src.get(f"{p}experts.{e}.down_proj").to(device, dtype)
        if fused:
            g, u = _fold(g, post, cfg.norm_one_plus_w), _fold(u, post, cfg.norm_one_plus_w)
        gus.append(L.interleave_gate_up(g, u, bn))
        downs.append(L.pad_rows(d, 128))
    router = src.get(p + "router").to(device, dtype)
    if fused:
        router = _fold(router, post, cfg.norm_one_plus_w)
    router = L.pad_rows(router, 128).contiguous()
    rb = src.get(p + "router_bias").float().to(device) if src.has(p + "router_bias") else None
    w_gu, w_dn = torch.cat(gus, 0).contiguous(), torch.cat(downs, 0).contiguous()
    if expert_quant in ("mxfp8", "nvfp4"):
        # expert stacks as block-scaled operands (MXFP8: e4m3 + ue8m0 per 32; NVFP4: e2m1 + ue4m3 per 16): the grouped
        # GEMMs then run on the block-scaled tensor-core kinds and half / a quarter of the bytes cross HBM
        from ..ops import blockscale as B
        mult = 128 if expert_quant == "mxfp8" else 256
        if cfg.hidden_size % mult or inter % mult or (2 * inter) % 128 or w_dn.shape[0] // max(e1 - e0, 1) % 128:
            raise ValueError(f"{expert_quant} experts need hidden / intermediate sizes that are multiples of {mult}")
        w_gu, w_dn = B.quantize(w_gu.float(), expert_quant), B.quantize(w_dn.float(), expert_quant)
    lw = MoeLayerWeights(router=router, router_bias=rb, w_gate_up=w_gu, w_down=w_dn, glu_bn=bn, e0=e0, e_local=e1 - e0,
                         inter=inter, cfg=cfg, fused=fused, ep=ep, tp_experts=tp_experts,
                         bs_fmt=expert_quant if expert_quant in ("mxfp8", "nvfp4") else None)
    if cfg.num_shared_experts and src.has(p + "shared_expert.gate_proj"):
        g = src.get(p + "shared_expert.gate_proj").to(device, dtype)
        u = src.get(p + "shared_expert.up_proj").to(device, dtype)
        if fused:
            g, u = _fold(g, post, cfg.norm_one_plus_w), _fold(u, post, cfg.norm_one_plus_w)
        lw.shared_bn = 256 if g.shape[0] % 128 == 0 else 128
        lw.shared_gate_up = L.interleave_gate_up(g, u, lw.shared_bn)
        lw.shared_down = L.pad_rows(src.get(p + "shared_expert.down_proj").to(device, dtype), 128).contiguous()
    return lw


class PagedExperts:
    """The expert stacks of one MoE layer in (pinned) host memory with ``slots`` experts resident on the device.

    ``ensure(experts)`` makes a set of experts resident (least recently used slots are reused; loads go through the
    layer's ``ExpertFaultHandler``, so every miss is counted and retried like a page fault); ``slot_map`` gives the
    device tensor expert -> slot for the resident ones (``slots`` = not resident, which the grouped GEMMs skip);
    ``after_gate`` feeds the cross-layer prefetcher, which loads the experts it expects next into slots the current
    step does not need. Reference: expert weight paging, fault handler and prefetch after the gate
    (src/scheduler/weight_paging.rs:26-601, src/moe/fault_handler.rs, src/moe/prefetch.rs)."""

    def __init__(self, layer: MoeLayerWeights, layer_index: int, slots: int, pager=None, cpu_experts: bool = False,
                 max_cpu_ratio: float = 0.2):
        from ..moe.routing import ExpertThermalTracker
        self.cpu_experts, self.max_cpu_ratio = bool(cpu_experts), float(max_cpu_ratio)
        self.thermal = ExpertThermalTracker(layer.e_local)
        self.last_plan = None
        self.glu_bn = layer.glu_bn
        if layer.bs_fmt is not None or layer.ep is not None or layer.tp_experts is not None:
            raise ValueError("paged experts: bf16 expert stacks on one rank only")
        from ..moe.residency import ExpertFaultHandler
        self.layer_index, self.pager = layer_index, pager
        self.e_local = layer.e_local
        self.slots = max(1, min(int(slots), layer.e_local))
        dev = layer.w_gate_up.device
        self.rows_gu = layer.w_gate_up.shape[0] // layer.e_local
        self.rows_dn = layer.w_down.shape[0] // layer.e_local
        pin = dev.type == "cuda"
        self.host_gu = layer.w_gate_up.to("cpu").contiguous()
        self.host_dn = layer.w_down.to("cpu").contiguous()
        if pin:
            self.host_gu, self.host_dn = self.host_gu.pin_memory(), self.host_dn.pin_memory()
        self.dev_gu = torch.zeros((self.slots * self.rows_gu, layer.w_gate_up.shape[1]), dtype=layer.w_gate_up.dtype, device=dev)
        self.dev_dn = torch.zeros((self.slots * self.rows_dn, layer.w_down.shape[1]), dtype=layer.w_down.dtype, device=dev)
        layer.w_gate_up = layer.w_down = None          # the full stacks leave the device
        # the slots are the arena of a weight page table (one unit per expert): it keeps the LRU order, evicts, and
        # retries failed copies; pages of the wave being computed are pinned so that they cannot evict one another
        from ..scheduler.weight_paging import WeightPageTable
        self.table = WeightPageTable(self.slots, self._copy_in, max_retries=1)
        for e in range(self.e_local):
            self.table.add(self._key(e), 1)
        self.slot_of: dict = {}                        # resident expert -> slot
        self._map = torch.full((self.e_local,), self.slots, dtype=torch.int32, device=dev)
        self._protected: set = set()
        self.handler = ExpertFaultHandler(self._load)
        self.stats = {"hits": 0, "misses": 0, "evictions": 0, "prefetched": 0}

    def resident_bytes(self) -> int:
        return self.dev_gu.numel() * self.dev_gu.element_size() + self.dev_dn.numel() * self.dev_dn.element_size()

    def _key(self, e: int) -> str:
        return f"L{self.layer_index}.experts.{int(e)}"

    def _copy_in(self, page, slot: int):
        e = int(page.key.rsplit(".", 1)[1])
        self.dev_gu[slot * self.rows_gu:(slot + 1) * self.rows_gu].copy_(self.host_gu[e * self.rows_gu:(e + 1) * self.rows_gu],
                                                                        non_blocking=True)
        self.dev_dn[slot * self.rows_dn:(slot + 1) * self.rows_dn].copy_(self.host_dn[e * self.rows_dn:(e + 1) * self.rows_dn],
                                                                        non_blocking=True)

    def _load(self, layer_index: int, e: int):
        from ..scheduler.types import Tier
        slot = self.table.ensure_resident(self._key(e))
        for other in [x for x in self.slot_of if self.table.pages[self._key(x)].tier != Tier.L1_GPU]:
            del self.slot_of[other]                      # evicted by the table to make room
            self._map[other] = self.slots
            self.handler.evict(self.layer_index, other)
        self.slot_of[int(e)] = slot
        self._map[int(e)] = slot
        self.stats["evictions"] = self.table.stats["evictions"]

    def _pin(self, experts):
        for e in self._protected:
            self.table.pages[self._key(e)].pinned = False
        self._protected = set(int(e) for e in experts)
        for e in self._protected:
            self.table.pages[self._key(e)].pinned = True

    def ensure(self, experts):
        """Make these (local) experts resident; they cannot evict one another."""
        if len(experts) > self.slots:
            raise ValueError(f"{len(experts)} experts do not fit {self.slots} slots")
        self._pin(experts)
        for e in self._protected:
            if e in self.slot_of:
                self.table.ensure_resident(self._key(e))   # a hit: refreshes its place in the LRU order
                self.stats["hits"] += 1
            else:
                self.stats["misses"] += 1
                if not self.handler.ensure(self.layer_index, e):
                    raise RuntimeError(f"layer {self.layer_index}: expert {e} could not be loaded: "
                                       f"{self.handler.errors.get((self.layer_index, e))}")

    def slot_map(self, experts) -> torch.Tensor:
        """[e_local] int32 on the device: slot of each of ``experts``, ``slots`` for every other expert (resident or
        not: a wave computes only its own experts)."""
        m = torch.full_like(self._map, self.slots)
        idx = torch.as_tensor(list(experts), dtype=torch.long, device=m.device)
        if idx.numel():
            m[idx] = self._map[idx]
        return m

    def prefetch(self, e: int) -> bool:
        """Load an expert the prefetcher expects, into a free slot or over an expert the current wave does not need."""
        if e in self.slot_of:
            return False
        if len(self.slot_of) >= self.slots and all(x in self._protected for x in self.slot_of):
            return False
        if self.handler.ensure(self.layer_index, int(e)):
            self.stats["prefetched"] += 1
            return True
        return False

    def after_gate(self, ids):
        if self.pager is not None:
            self.pager.after_gate(self.layer_index, ids)

    def run_on_host(self, e: int, src, row_ss, ids, w, acc, layer: MoeLayerWeights, model):
        """One expert's rows on the host, from the host copy of its weights (no weight transfer: only the few routed
        rows cross the bus, twice): acc[t] += w[t, k] * expert_e(src[t]) for every (t, k) routed to ``e``."""
        c = layer.cfg
        hit = (ids.long() == (e + layer.e0))                              # [T, k]
        tok = hit.any(1).nonzero().reshape(-1)
        if tok.numel() == 0:
            return
        x = src.index_select(0, tok).float().cpu()
        if row_ss is not None:                                            # fused layout: the norm weight is in the weights
            ss = row_ss.index_select(0, tok).float().reshape(tok.numel(), -1).sum(-1).cpu()
            x = x * torch.rsqrt(ss / c.hidden_size + c.rms_norm_eps)[:, None]
        gu = self.host_gu[e * self.rows_gu:(e + 1) * self.rows_gu].float()
        g, u = L.deinterleave_gate_up(gu, self.glu_bn)
        a = L._act_ref(x @ g.t(), model.act_id) * (x @ u.t())
        dn = self.host_dn[e * self.rows_dn:(e + 1) * self.rows_dn].float()[:c.hidden_size]
        y = a[:, :dn.shape[1]] @ dn.t()
        wt = (w.float() * hit).sum(1).index_select(0, tok).cpu()
        acc.index_add_(0, tok, (y * wt[:, None]).to(acc.dtype).to(acc.device))
        self.stats["host_rows"] = self.stats.get("host_rows", 0) + int(tok.numel())


class ExpertPager:
    """All paged MoE layers of a model and the prefetcher that links them: the experts chosen at layer l predict the
    experts of the next layers (transition counts learnt while serving), which are loaded ahead of their gate."""

    def __init__(self, num_layers: int, num_experts: int, depth: int = 1, top: int = 4):
        from ..moe.residency import ExpertPrefetcher
        self.layers: dict = {}
        self.prefetcher = ExpertPrefetcher(num_layers, num_experts, depth=depth, top=top)

    def add(self, layer_index: int, paged: PagedExperts):
        self.layers[layer_index] = paged
        paged.pager = self

    def after_gate(self, layer_index: int, ids):
        host = ids.detach().to("cpu")
        self.prefetcher.observe(layer_index, host)
        for req in self.prefetcher.predict(layer_index, host):
            tgt = self.layers.get(req.layer)
            if tgt is not None:
                tgt._pin(())
                tgt.prefetch(req.expert)

    def stats(self) -> dict:
        out = {"hits": 0, "misses": 0, "evictions": 0, "prefetched": 0, "faults": 0, "resident_bytes": 0}
        for pg in self.layers.values():
            for k in ("hits", "misses", "evictions", "prefetched"):
                out[k] += pg.stats[k]
            out["faults"] += pg.handler.stats["faults"]
            out["resident_bytes"] += pg.resident_bytes()
        return out
