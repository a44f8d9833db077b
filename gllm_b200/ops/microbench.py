"""Kernel microbenchmarks: ``python -m gllm_b200.ops.microbench --op <name> [--iters N]``.

Each op runs a small, fixed case (inputs larger than L2, a few hundred MB on the device at most) so it can
also be captured with ``ncu`` in a minute or two. Timing uses CUDA events on the launching stream after
warm-up; the achieved fraction of the measured peaks (``MEASURED_PEAKS.json`` at the repository root if
present) is printed as JSON.

ops: bsgemm_mxfp8  bsgemm_nvfp4  gemm_prefill  gemm_prefill_glu  gemm_prefill_residual  gemm_prefill_qkv  gemm_decode  gemm_decode_trace  gemm_glu  gemm_qkv  decode_attn  prefill_attn  sample  qgemm_fp8  qgemm_fp4  qgemm_int4
     mla_attn
"""
from __future__ import annotations

import argparse
import json
import os
from pathlib import Path

import torch

from .. import ops


def _peaks():
    p = Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return d.get("hbm_gbs", 6650.0), d.get("bf16_tflops", 1590.0), "measured"
    return 6650.0, 1590.0, "fallback"


def _time(fn, iters, warmup=3):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    if os.environ.get("GLLM_BENCH_GRAPH", "0") == "1":
        # device time without per-call host overhead: `iters` calls captured in one CUDA graph
        g = torch.cuda.CUDAGraph()
        st = torch.cuda.Stream()
        with torch.cuda.stream(st):
            with torch.cuda.graph(g, stream=st):
                for _ in range(iters):
                    fn()
            g.replay()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            g.replay()
            e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / iters * 1e-3
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters * 1e-3  # seconds


def run(op: str, iters: int):
    dev = torch.device("cuda")
    hbm, tf, src = _peaks()
    torch.manual_seed(0)
    rnd = lambda *s, scale=1.0: (torch.randn(*s, device=dev) * scale).to(torch.bfloat16)
    out = {"op": op, "peaks": src}
    if op == "gemm_prefill":
        M, N, K = 8192, 8192, 4096
        a, w = rnd(M, K), rnd(N, K, scale=0.05)
        o = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
        t = _time(lambda: ops.gemm(a, w, out=o, bn=256), iters)
        out.update(shape=[M, N, K], us=t * 1e6, tflops=2 * M * N * K / t / 1e12, frac_of_bf16_peak=2 * M * N * K / t / 1e12 / tf)
    elif op in ("gemm_prefill_glu", "gemm_prefill_residual", "gemm_prefill_qkv"):
        # the epilogue variants at a prefill chunk (M = 8192), Qwen3-8B shapes
        M, K = 8192, 4096
        a = rnd(M, K)
        ss = a.float().pow(2).sum(-1, keepdim=True).contiguous()
        if op == "gemm_prefill_glu":
            I_ = 12288
            bn = int(os.environ.get("GLLM_GLU_BN", "0")) or __import__("gllm_b200.models.weights", fromlist=["x"]).glu_tile_width(I_)
            w = ops.interleave_gate_up(rnd(I_, K, scale=0.05), rnd(I_, K, scale=0.05), bn)
            o = torch.empty(M, I_, device=dev, dtype=torch.bfloat16)
            t = _time(lambda: ops.gemm_glu(a, w, out=o, row_ss=ss, norm_dim=K, eps=1e-6, bn=bn), iters)
            fl = 2 * M * 2 * I_ * K
            out.update(shape=[M, 2 * I_, K], bn=bn)
        elif op == "gemm_prefill_residual":
            N, K2 = 4096, 12288
            a2, w = rnd(M, K2), rnd(N, K2, scale=0.05)
            r = rnd(M, N)
            o = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
            t = _time(lambda: ops.gemm_residual(a2, w, r, out=o, bn=256), iters)
            fl = 2 * M * N * K2
            out.update(shape=[M, N, K2])
        else:
            nq, nkv = 32, 8
            w = rnd((nq + 2 * nkv) * 128, K, scale=0.05)
            kv = torch.zeros(M // 16 + 1, 2, nkv, 16, 128, device=dev, dtype=torch.bfloat16)
            q = torch.empty(M, nq * 128, device=dev, dtype=torch.bfloat16)
            pos = torch.arange(M, device=dev, dtype=torch.int32)
            inv = 1.0 / (1e6 ** (torch.arange(0, 128, 2, device=dev).double() / 128))
            ang = torch.arange(M, device=dev).double()[:, None] * inv[None]
            cos, sin = ang.cos().float().contiguous(), ang.sin().float().contiguous()
            qn = torch.ones(128, device=dev)
            t = _time(lambda: ops.gemm_qkv(a, w, n_q=nq, n_kv=nkv, q_out=q, kv_cache=kv, slot_mapping=pos, positions=pos,
                                           cos_t=cos, sin_t=sin, q_norm_w=qn, k_norm_w=qn, row_ss=ss, norm_dim=K, eps=1e-6), iters)
            fl = 2 * M * (nq + 2 * nkv) * 128 * K
            out.update(shape=[M, (nq + 2 * nkv) * 128, K])
        out.update(us=t * 1e6, tflops=fl / t / 1e12, frac_of_bf16_peak=fl / t / 1e12 / tf)
    elif op == "gemm_decode":
        # default: the down projection; GLLM_DEC_N / GLLM_DEC_K / GLLM_DEC_BN / GLLM_DEC_SPLITS reshape it
        M, N, K = 256, int(os.environ.get("GLLM_DEC_N", 4096)), int(os.environ.get("GLLM_DEC_K", 12288))
        bn, sp = int(os.environ.get("GLLM_DEC_BN", 256)), int(os.environ.get("GLLM_DEC_SPLITS", 0))
        ws = [rnd(N, K, scale=0.05) for _ in range(3)]
        a, r = rnd(M, K), rnd(M, N)
        o = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
        i = [0]
        out.update(bn=bn, splits=sp)

        def f():
            i[0] = (i[0] + 1) % 3
            ops.gemm_residual(a, ws[i[0]], r, out=o, bn=bn, splits=sp)
        t = _time(f, iters)
        byts = N * K * 2
        out.update(shape=[M, N, K], us=t * 1e6, weight_gbs=byts / t / 1e9, frac_of_hbm_peak=byts / t / 1e9 / hbm)
    elif op == "gemm_decode_trace":
        # SM-clock stamps of CTA 0's phases for one decode-shaped residual GEMM (same GLLM_DEC_* knobs; GLLM_PAIR=1 for
        # the CTA-pair kernel); weights rotate over three sets so that they stream from HBM
        import ctypes
        from . import _native as nv
        lib = nv.lib()
        lib.gllm_gemm_set_trace.argtypes = [ctypes.c_void_p]
        lib.gllm_gemm_set_trace.restype = None
        M, N, K = 256, int(os.environ.get("GLLM_DEC_N", 4096)), int(os.environ.get("GLLM_DEC_K", 12288))
        bn, sp = int(os.environ.get("GLLM_DEC_BN", 256)), int(os.environ.get("GLLM_DEC_SPLITS", 0))
        ws = [rnd(N, K, scale=0.05) for _ in range(3)]
        a, r = rnd(M, K), rnd(M, N)
        o = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
        i = [0]
        glu = os.environ.get("GLLM_DEC_EPI", "residual") == "glu"    # N counts gate + up rows then
        store32 = os.environ.get("GLLM_DEC_EPI", "residual") == "store_f32"   # the lm_head: fp32 logits
        ss = a.float().pow(2).sum(-1, keepdim=True).contiguous()
        o32 = torch.empty(M, N, device=dev, dtype=torch.float32) if store32 else None

        def f():
            i[0] = (i[0] + 1) % 3
            if store32:
                ops.gemm(a, ws[i[0]], out=o32, out_dtype=torch.float32, row_ss=ss, norm_dim=K, eps=1e-6, bn=bn, splits=sp)
            elif glu:
                ops.gemm_glu(a, ws[i[0]], out=o[:, :N // 2], row_ss=ss, norm_dim=K, eps=1e-6, bn=bn, splits=sp)
            else:
                ops.gemm_residual(a, ws[i[0]], r, out=o, bn=bn, splits=sp)
        os.environ["GLLM_BENCH_GRAPH"] = "1"
        t = _time(f, iters)
        tr = torch.zeros(12, dtype=torch.int64, device=dev)
        lib.gllm_gemm_set_trace(tr.data_ptr())
        f()
        torch.cuda.synchronize()
        lib.gllm_gemm_set_trace(None)
        st = tr.tolist()
        names = ["set_up", "first_stage", "main_loop", "accumulator_ready", "epilogue_or_dump", "drain", "grid_barrier",
                 "reduce"]
        out.update(shape=[M, N, K], bn=bn, splits=sp, us=t * 1e6,
                   clocks={n: (st[j + 1] - st[j] if st[j + 1] and st[j] else 0) for j, n in enumerate(names)})
    elif op == "gemm_glu":
        M, I, K = 256, int(os.environ.get("GLLM_GLU_I", 12288)), 4096    # GLLM_GLU_I=1536: one rank's share at TP8
        from ..models.weights import glu_tile_width
        bn = int(os.environ.get("GLLM_GLU_BN", "0")) or glu_tile_width(I)
        ws = [ops.interleave_gate_up(rnd(I, K, scale=0.05), rnd(I, K, scale=0.05), bn) for _ in range(2)]
        a = rnd(M, K)
        ss = a.float().pow(2).sum(-1, keepdim=True).contiguous()
        o = torch.empty(M, I, device=dev, dtype=torch.bfloat16)
        i = [0]

        def f():
            i[0] ^= 1
            ops.gemm_glu(a, ws[i[0]], out=o, row_ss=ss, norm_dim=K, eps=1e-6, bn=bn)
        t = _time(f, iters)
        byts = 2 * I * K * 2
        out.update(shape=[M, 2 * I, K], bn=bn, us=t * 1e6, weight_gbs=byts / t / 1e9, frac_of_hbm_peak=byts / t / 1e9 / hbm)
    elif op == "gemm_qkv":
        M, K, nq, nkv = int(os.environ.get("GLLM_QKV_M", 2048)), 4096, 32, 8
        a, w = rnd(M, K), rnd((nq + 2 * nkv) * 128, K, scale=0.05)
        ss = a.float().pow(2).sum(-1, keepdim=True).contiguous()
        kv = torch.zeros(M // 16 + 1, 2, nkv, 16, 128, device=dev, dtype=torch.bfloat16)
        q = torch.empty(M, nq * 128, device=dev, dtype=torch.bfloat16)
        pos = torch.arange(M, device=dev, dtype=torch.int32)
        inv = 1.0 / (1e6 ** (torch.arange(0, 128, 2, device=dev).double() / 128))
        ang = torch.arange(M, device=dev).double()[:, None] * inv[None]
        cos, sin = ang.cos().float().contiguous(), ang.sin().float().contiguous()
        qn = torch.ones(128, device=dev)
        t = _time(lambda: ops.gemm_qkv(a, w, n_q=nq, n_kv=nkv, q_out=q, kv_cache=kv, slot_mapping=pos, positions=pos,
                                       cos_t=cos, sin_t=sin, q_norm_w=qn, k_norm_w=qn, row_ss=ss, norm_dim=K, eps=1e-6),
                  iters)
        fl = 2 * M * (nq + 2 * nkv) * 128 * K
        out.update(shape=[M, (nq + 2 * nkv) * 128, K], us=t * 1e6, tflops=fl / t / 1e12, frac_of_bf16_peak=fl / t / 1e12 / tf)
    elif op.startswith("qgemm_"):
        # decode-shaped weight streaming: the quantised codes are what crosses HBM
        from . import quant_gemm as Q
        mode = op.split("_", 1)[1]
        M, N, K = 256, 12288, 4096
        group = 16 if mode == "fp4" else 32
        ws = [Q.quantize(torch.randn(N, K) * 0.05, mode, group).to(dev) for _ in range(3)]
        a = rnd(M, K)
        o = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
        i = [0]

        def f():
            i[0] = (i[0] + 1) % 3
            Q.qgemm(a, ws[i[0]], out=o)
        t = _time(f, iters)
        byts = ws[0].nbytes()
        dense = N * K * 2
        out.update(shape=[M, N, K], mode=mode, group=group, us=t * 1e6, weight_bytes=byts, weight_gbs=byts / t / 1e9,
                   frac_of_hbm_peak=byts / t / 1e9 / hbm, bf16_equivalent_gbs=dense / t / 1e9,
                   tflops=2 * M * N * K / t / 1e12)
    elif op in ("ar_ll_world1", "ar_push_world1", "ar_pull_world1"):
        # the fused row-parallel GEMM + all-reduce kernel on ONE GPU (world size 1, ordinary device memory): the whole
        # protocol runs (self-validating slots, receive slots / tile flags / done words, or buffers / arrival counters) without a peer, which
        # is the form that can sit under a profiler. Decode-sized o_proj of a TP-8 shard by default.
        from ..parallel.tensor_parallel import single_gpu_context
        M, N, K = [int(v) for v in os.environ.get("GLLM_AR_SHAPE", "256,4096,512").split(",")]
        tp = single_gpu_context(dev, hidden=N, max_tokens=max(M, 256), mode={"ar_ll_world1": "ll_p2p", "ar_push_world1": "fused_p2p"}.get(op, "pull_p2p"))
        ws = [rnd(N, K, scale=0.05) for _ in range(8)]
        a = rnd(M, K)
        bufs = tp.workspace_buffers(M) if op == "ar_push_world1" else None
        x = bufs["x"] if bufs else rnd(M, N)
        ss = (bufs["ss_a"].reshape(-1)[:M * (N // 256)].view(M, N // 256) if bufs else torch.zeros(M, N // 256, device=dev))
        i = [0]

        def f():
            i[0] = (i[0] + 1) % 8
            tp.gemm_allreduce_residual(a, ws[i[0]], x, ss, None)
        t = _time(f, iters)
        out.update(shape=[M, N, K], form=tp.form, us=t * 1e6, weight_gbs=N * K * 2 / t / 1e9)
    elif op.startswith("bsgemm_"):
        # block-scaled tensor-core GEMM (both operands MXFP8 / NVFP4, hardware scale factors). Shape from GLLM_BS_SHAPE
        # ("M,N,K"); default: the decode-sized gate/up projection. GLLM_BS_QUANT=1 adds the activation quantisation.
        from . import blockscale as B
        fmt = op.split("_", 1)[1]
        M, N, K = [int(v) for v in os.environ.get("GLLM_BS_SHAPE", "256,12288,4096").split(",")]
        bn = int(os.environ.get("GLLM_BS_BN", "128"))
        nw = 3 if N * K <= (1 << 27) else 1
        ws = [B.quantize(torch.randn(N, K) * 0.05, fmt).to(dev) for _ in range(nw)]
        a = rnd(M, K)
        aq = B.quantize_act(a, fmt, tensor_scale=0.02)
        o = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
        with_quant = os.environ.get("GLLM_BS_QUANT", "0") == "1"
        i = [0]

        def f():
            i[0] = (i[0] + 1) % nw
            if with_quant:
                B.quantize_act(a, fmt, out=aq, tensor_scale=0.02)
            B.gemm(aq, ws[i[0]], out=o, bn=bn)
        t = _time(f, iters)
        byts = ws[0].nbytes()
        out.update(shape=[M, N, K], fmt=fmt, bn=bn, with_quant=with_quant, us=t * 1e6, weight_bytes=byts,
                   weight_gbs=byts / t / 1e9, frac_of_hbm_peak=byts / t / 1e9 / hbm, tflops=2 * M * N * K / t / 1e12,
                   frac_of_bf16_peak=2 * M * N * K / t / 1e12 / tf)
    elif op == "mla_attn":
        from . import mla as MLA
        nh, d_c, d_r = 16, 512, 64
        B, ctx = int(os.environ.get("GLLM_MLA_BATCH", 256)), 1024
        pages = B * ctx // 16
        cache = rnd(pages, 16, d_c + d_r, scale=0.3)
        q = rnd(B, nh * (d_c + d_r), scale=0.3)
        bt = torch.arange(pages, device=dev, dtype=torch.int32).reshape(B, ctx // 16)
        idx = torch.arange(B, device=dev, dtype=torch.int32)
        one = torch.ones(B, device=dev, dtype=torch.int32)
        cl = torch.full((B,), ctx, device=dev, dtype=torch.int32)
        o = torch.empty(B, nh * d_c, device=dev, dtype=torch.bfloat16)
        if os.environ.get("GLLM_MLA_CUDA_CORES", "0") == "1":
            t = _time(lambda: MLA.latent_attention(q, cache, bt, idx, one, cl, idx, n_heads=nh, d_v=d_c, scale=0.04, out=o), iters)
        else:
            t = _time(lambda: MLA.latent_decode(q, cache, bt, cl, n_heads=nh, scale=0.04, out=o), iters)
        byts = cache.numel() * 2
        fl = 2 * B * nh * ctx * (2 * d_c + d_r)
        out.update(shape=dict(batch=B, heads=nh, ctx=ctx, d_c=d_c, d_rope=d_r), us=t * 1e6, kv_gbs=byts / t / 1e9,
                   frac_of_hbm_peak=byts / t / 1e9 / hbm, tflops=fl / t / 1e12)
    elif op == "mla_prefill":
        # one prefill chunk of the absorbed attention: S prompts of L tokens, 16 heads (DeepSeek-V3 at eight ranks)
        from . import mla as MLA
        nh, d_c, d_r = 16, 512, 64
        S, Lq = int(os.environ.get("GLLM_MLA_SEQS", 2)), int(os.environ.get("GLLM_MLA_LEN", 2048))
        T = S * Lq
        pages = T // 16
        cache = rnd(pages, 16, d_c + d_r, scale=0.3)
        q = rnd(T, nh * (d_c + d_r), scale=0.3)
        bt = torch.arange(pages, device=dev, dtype=torch.int32).reshape(S, Lq // 16)
        qs = torch.arange(S, device=dev, dtype=torch.int32) * Lq
        ql = torch.full((S,), Lq, device=dev, dtype=torch.int32)
        row_seq = torch.repeat_interleave(torch.arange(S, device=dev, dtype=torch.int32), Lq)
        pos = torch.arange(Lq, device=dev, dtype=torch.int32).repeat(S)
        o = torch.empty(T, nh * d_c, device=dev, dtype=torch.bfloat16)
        if os.environ.get("GLLM_MLA_CUDA_CORES", "0") == "1":
            t = _time(lambda: MLA.latent_attention(q, cache, bt, qs, ql, ql, row_seq, n_heads=nh, d_v=d_c, scale=0.04, out=o), iters)
        else:
            t = _time(lambda: MLA.latent_prefill(q, cache, bt, row_seq, pos, ql, n_heads=nh, scale=0.04, max_ctx=Lq, out=o), iters)
        fl = 2 * S * nh * (Lq * (Lq + 1) // 2) * (2 * d_c + d_r)
        out.update(shape=dict(seqs=S, len=Lq, heads=nh, d_c=d_c, d_rope=d_r), us=t * 1e6, tflops=fl / t / 1e12,
                   frac_of_bf16_peak=fl / t / 1e12 / tf, cuda_cores=os.environ.get("GLLM_MLA_CUDA_CORES", "0") == "1")
    elif op in ("decode_attn", "prefill_attn"):
        nq, nkv, D = 32, 8, 128
        if op == "decode_attn":
            # defaults: the committed case. GLLM_ATTN_* reshape it, e.g. one rank's share under 8-way tensor
            # parallelism: GLLM_ATTN_NQ=4 GLLM_ATTN_NKV=1 GLLM_ATTN_BATCH=256 GLLM_ATTN_RAGGED=1 GLLM_ATTN_PPS=16
            nq, nkv = int(os.environ.get("GLLM_ATTN_NQ", nq)), int(os.environ.get("GLLM_ATTN_NKV", nkv))
            B, ctx = int(os.environ.get("GLLM_ATTN_BATCH", 64)), 2048
            pps = int(os.environ.get("GLLM_ATTN_PPS", 1 << 20))
            pages = B * ctx // 16
            kv = torch.randn(pages, 2, nkv, 16, D, device=dev).to(torch.bfloat16)
            fp8 = os.environ.get("GLLM_ATTN_FP8", "0") == "1"      # e4m3 cache, one byte per value
            if fp8:
                kv = (kv.float() / 0.05).to(torch.float8_e4m3fn)
            bt = torch.randperm(pages, device=dev).to(torch.int32).reshape(B, ctx // 16).contiguous()
            if os.environ.get("GLLM_ATTN_RAGGED", "0") == "1":
                cl = torch.randint(128, ctx + 1, (B,), device=dev).to(torch.int32)
            else:
                cl = torch.full((B,), ctx, dtype=torch.int32, device=dev)
            q = rnd(B, nq * D)
            o = torch.empty_like(q)
            max_splits = max(1, -(-(ctx // 16) // pps))
            wsp = ops.DecodeWorkspace(B, nq, nkv, max_splits, dev)
            t = _time(lambda: ops.paged_decode(q, kv, bt, cl, n_q=nq, n_kv=nkv, out=o, workspace=wsp,
                                               pages_per_split=pps, kv_scale=0.05), iters)
            byts = int(cl.sum().item()) * 2 * nkv * D * kv.element_size()
            out.update(batch=B, ctx=ctx, n_q=nq, n_kv=nkv, pages_per_split=pps, kv_dtype=str(kv.dtype).split(".")[-1], us=t * 1e6, kv_gbs=byts / t / 1e9,
                       frac_of_hbm_peak=byts / t / 1e9 / hbm)
        else:
            S, L = 8, 2048
            pages = S * L // 16
            kv = torch.randn(pages, 2, nkv, 16, D, device=dev).to(torch.bfloat16)
            bt = torch.arange(pages, device=dev, dtype=torch.int32).reshape(S, L // 16).contiguous()
            q = rnd(S * L, nq * D)
            o = torch.empty_like(q)
            qs = torch.arange(S, device=dev, dtype=torch.int32) * L
            ql = torch.full((S,), L, dtype=torch.int32, device=dev)
            t = _time(lambda: ops.paged_prefill(q, kv, bt, qs, ql, ql, max_q_len=L, n_q=nq, n_kv=nkv, out=o), iters)
            fl = 4 * S * L * L * D * nq / 2
            out.update(seqs=S, len=L, us=t * 1e6, tflops=fl / t / 1e12, frac_of_bf16_peak=fl / t / 1e12 / tf)
    elif op == "sample":
        B, V = 256, 151936
        lg = torch.randn(B, V, device=dev)
        params = torch.tensor([0.7, 50, 0.9, 0], device=dev).repeat(B, 1).contiguous()
        t = _time(lambda: ops.sample(lg, params, seed=1), iters)
        out.update(batch=B, vocab=V, us=t * 1e6, logits_gbs=B * V * 4 / t / 1e9)
    else:
        raise SystemExit(f"unknown op {op}")
    from . import _native as nv
    out["device_error"] = nv.device_error()
    print(json.dumps(out))
    return out


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--op", required=True)
    ap.add_argument("--iters", type=int, default=10)
    a = ap.parse_args()
    run(a.op, a.iters)
