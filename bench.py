#!/usr/bin/env python
"""Headline benchmark: decode tokens/s of the Qwen3-8B-shape dense decoder (bf16) under continuous
batching of 256 concurrent synthetic requests (prompt lengths uniform 128-2048, 16-token KV pages,
a 512-token shared prefix on half of the requests), tensor-parallel over N GPUs of one node.

    python bench.py --gpus 1 --steps 32 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W

A "step" is one decode iteration of the serving engine over all running sequences. Two numbers are
reported: ``value`` is device-timed (CUDA events around K replays of the captured decode step, max over
ranks); ``e2e`` times the same K steps through the public engine API, including every step's pinned-host
-> device upload of scheduler inputs and the device -> host read of the sampled tokens.
Rank 0 prints one JSON line.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=32)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="qwen3-8b")
    ap.add_argument("--concurrency", type=int, default=256)
    ap.add_argument("--min-prompt", type=int, default=128)
    ap.add_argument("--max-prompt", type=int, default=2048)
    ap.add_argument("--output-tokens", type=int, default=256)
    ap.add_argument("--shared-prefix", type=int, default=512)
    ap.add_argument("--tp-mode", default="auto", choices=["auto", "ll", "ll_p2p", "fused", "fused_p2p", "pull", "nccl"])
    ap.add_argument("--parallel", default="tp",
                    help="tp (tensor parallel over all GPUs, the headline), ep (data-parallel attention + expert-parallel "
                         "MoE, engines in lockstep), or tpXppY (X-way tensor parallel stages of a Y-stage pipeline)")
    ap.add_argument("--weight-quant", default=None, choices=[None, "mxfp8", "nvfp4"],
                    help="linear weights (and activations) block-scaled on the tensor cores")
    ap.add_argument("--expert-quant", default=None, choices=[None, "mxfp8", "nvfp4"], help="MoE expert weights block-scaled")
    ap.add_argument("--no-graphs", action="store_true")
    ap.add_argument("--sequence-parallel", action="store_true",
                    help="tensor parallel with the residual stream sharded by rows (reduce-scatter / all-gather forms)")
    ap.add_argument("--kv-dtype", default="bf16", choices=["bf16", "fp8"],
                    help="fp8: e4m3 KV cache (half the KV bytes); not the headline configuration, reported as invalid for it")
    ap.add_argument("--op-breakdown", action="store_true",
                    help="after the timed regions, time every op of one captured decode step with in-graph events")
    ap.add_argument("--layers", type=int, default=0, help="debug only: a value other than 0 marks the result invalid")
    ap.add_argument("--no-baseline", action="store_true",
                    help="skip the NCCL baseline arm (unfused GEMM + ncclAllReduce) that vs_baseline is measured against")
    ap.add_argument("--no-tp1-check", action="store_true",
                    help="skip the comparison of greedy tokens with a single-GPU run of the same model on rank 0")
    return ap.parse_args()


REFERENCE_UNAVAILABLE = (
    "reference is a Rust-nightly crate whose kernels and NCCL layer live in two sibling repositories "
    "(../gllm-kernels, ../gllm-nccl) that are not present; no Rust toolchain in this image, so pip cannot build it")


class ClockSampler:
    """Samples SM clocks / throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu, self.lines, self.proc = gpu_index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.gpu)], stdout=subprocess.PIPE, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            pass
        sm, mx, reasons, power = [], [], set(), []
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2])); power.append(float(f[3]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(power) if power else None, "samples": len(sm), "reasons": sorted(reasons)}


def make_prompts(n, lo, hi, shared_prefix, vocab, seed=1234):
    import numpy as np
    rng = np.random.RandomState(seed)
    prefix = rng.randint(0, vocab, size=shared_prefix).tolist()
    prompts = []
    for i in range(n):
        ln = int(rng.randint(lo, hi + 1))
        if i % 2 == 0 and ln > shared_prefix:
            prompts.append(prefix + rng.randint(0, vocab, size=ln - shared_prefix).tolist())
        else:
            prompts.append(rng.randint(0, vocab, size=ln).tolist())
    return prompts


def main():
    args = parse_args()
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": REFERENCE_UNAVAILABLE}))
        return 0

    import numpy as np
    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            # relaunch under torchrun so that `python bench.py --gpus N` works on its own
            port = 29500 + (os.getpid() % 2000)
            cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
                   "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.abspath(__file__)] + sys.argv[1:]
            return subprocess.call(cmd)
        raise SystemExit(f"WORLD_SIZE={world} does not match --gpus {args.gpus}")
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (sm_100a)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    from gllm_b200.engine.executor import EngineConfig, LLMEngine
    from gllm_b200.models.config import preset
    from gllm_b200.models.decoder import DecoderModel
    from gllm_b200.models.weights import RandomWeights
    from gllm_b200.ops import _native as nv

    cfg = preset(args.model)
    if args.layers:
        cfg.num_layers = args.layers
    # ---- parallel layout: ranks = pipeline stage * tp + tensor-parallel index ----
    import re
    par = args.parallel.lower()
    tp_size, pp_size, ep_mode = world, 1, False
    if par == "ep":
        tp_size, ep_mode = 1, world > 1
    elif par != "tp":
        m = re.fullmatch(r"tp(\d+)(?:pp(\d+))?", par)
        if not m:
            raise SystemExit(f"--parallel {args.parallel!r}: expected tp, ep or tpXppY")
        tp_size, pp_size = int(m.group(1)), int(m.group(2) or 1)
        if tp_size * pp_size != world:
            raise SystemExit(f"--parallel {args.parallel}: {tp_size} x {pp_size} != {world} GPUs")
    stage, tpi = rank // tp_size, rank % tp_size
    max_len = args.max_prompt + args.output_tokens + 16
    tp = ep = pp_ctx = None
    lockstep = None
    if tp_size > 1:
        from gllm_b200.parallel.tensor_parallel import TPContext
        tp_group = None
        if pp_size > 1:      # one tensor-parallel group per pipeline stage (creating a group is collective over the world)
            for st in range(pp_size):
                g = dist.new_group(list(range(st * tp_size, (st + 1) * tp_size)))
                if st == stage:
                    tp_group = g
        tp = TPContext(tpi, tp_size, dev, mode=args.tp_mode, max_tokens=8192, hidden=cfg.hidden_size, group=tp_group)
    if pp_size > 1:
        from gllm_b200.engine.pp import build_pipeline
        from gllm_b200.parallel.comm import CommHandle
        pp_ctx = build_pipeline(CommHandle.from_env("nccl", device=dev), pp=pp_size, tp=tp_size)
    if ep_mode:
        from gllm_b200.parallel.expert_parallel import EPContext
        ep = EPContext(rank, world, dev, num_experts=cfg.num_experts, hidden=cfg.hidden_size,
                       top_k=cfg.num_experts_per_tok, max_tokens=8192, mode="fused")
        lockstep = dist.group.WORLD
    layers = None
    if pp_size > 1:
        from gllm_b200.parallel.pipeline import PipelineConfig
        layers = PipelineConfig(num_layers=cfg.num_layers, num_stages=pp_size).stage_ranges()[stage]
    src = RandomWeights(cfg, dev, torch.bfloat16, seed=0)
    kv_kw = dict(kv_dtype=torch.float8_e4m3fn, kv_scale=0.05) if args.kv_dtype == "fp8" else {}
    model = DecoderModel(cfg, src, device=dev, dtype=torch.bfloat16, tp=tp, max_positions=max_len, layers=layers, ep=ep,
                         weight_quant=args.weight_quant, expert_quant=args.expert_quant,
                         sequence_parallel=bool(args.sequence_parallel and tp is not None), **kv_kw)
    # data-parallel attention: every rank serves its own share of the requests
    conc_total = args.concurrency
    if ep_mode:
        args.concurrency = max(1, args.concurrency // world)
    ecfg = EngineConfig(max_num_seqs=args.concurrency, max_model_len=max_len, max_batch_tokens=8192,
                        prefill_chunk=8192, use_cuda_graphs=not args.no_graphs)
    ecfg.num_pages = args.concurrency * ((max_len + 15) // 16) + 64
    engine = LLMEngine(model, ecfg, lockstep_group=lockstep, pp=pp_ctx)
    engine.precapture()        # decode graphs for every batch bucket, as a server does at start-up (not part of TTFT)
    prompts = make_prompts(conc_total, args.min_prompt, args.max_prompt, args.shared_prefix, cfg.vocab_size)
    if ep_mode:
        prompts = prompts[rank::world]

    # ---- phase 0 (N > 1): the tensor-parallel engine against the single-GPU model ----
    # The TP engine generates 8 greedy tokens for 8 prompts. The single-GPU model of the same weights then scores the
    # same sequences teacher-forced (one forward over prompt + generated tokens, logits at the 64 generated positions),
    # so a token that flipped between two near-equal logits does not compound. With random-init weights the logits
    # are close to flat (the gap between the two largest of 150 k is about 0.2 standard deviations), so the check is on
    # the GAP: every token the TP engine chose must lie within 0.25 standard deviations of the single-GPU maximum
    # (a wrong kernel picks tokens about 4-5 standard deviations below it) and most must be the exact argmax.
    tp1_check = None
    if world > 1 and par == "tp" and not args.no_tp1_check:
        from gllm_b200.engine.batch import ForwardBatch
        check_prompts = make_prompts(8, 24, 96, 16, cfg.vocab_size, seed=4321)
        got = [r.token_ids for r in engine.generate_batch(check_prompts, max_tokens=8, temperature=0.0, eos_ids=[])]
        if rank == 0:
            ref_model = DecoderModel(cfg, src, device=dev, dtype=torch.bfloat16, max_positions=max_len, **kv_kw)
            exact = first = 0
            gaps = []
            for pr, g in zip(check_prompts, got):
                ids = list(pr) + list(g[:-1])
                n = len(ids)
                rows = [len(pr) - 1 + i for i in range(len(g))]
                kv = ref_model.alloc_kv_cache((n + 15) // 16 + 1)
                i32 = dict(dtype=torch.int32, device=dev)
                fb = ForwardBatch(token_ids=torch.tensor(ids, **i32), positions=torch.arange(n, **i32),
                                  slot_mapping=torch.arange(n, **i32),
                                  block_tables=torch.arange((n + 15) // 16, **i32)[None],
                                  ctx_lens=torch.tensor([n], **i32), q_start=torch.tensor([0], **i32),
                                  q_len=torch.tensor([n], **i32), max_q_len=n,
                                  logits_rows=torch.tensor(rows, dtype=torch.int64, device=dev))
                lg = ref_model.forward(fb, kv).float()[:, :cfg.vocab_size]
                for i, tok in enumerate(g):
                    row = lg[i]
                    gaps.append(float((row.max() - row[int(tok)]) / row.std()))
                    hit = int(int(row.argmax()) == int(tok))
                    exact += hit
                    first += hit if i == 0 else 0
                del kv
            tp1_check = {"method": "teacher-forced single-GPU logits at the generated positions",
                         "tokens_equal": exact, "tokens_total": len(gaps), "first_tokens_equal": first, "prompts": 8,
                         "max_gap_sigma": round(max(gaps), 4), "mean_gap_sigma": round(sum(gaps) / len(gaps), 5)}
            del ref_model
            torch.cuda.empty_cache()
        dist.barrier()
        for k in engine.stats:          # the check's prefill / decode work is not part of the measured workload
            engine.stats[k] = 0

    prefix_hits0 = int(engine.batcher.prefix_hits)
    W, K = max(args.warmup, 3), args.steps
    # every request generates the configured number of tokens; the timed window sits in the middle of it
    budget_tokens = max(args.output_tokens, W + K + 4)
    center_steps = max(0, (budget_tokens - K) // 2 - W)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    # ---- phase 1: admit + prefill everything (untimed for the decode metric; gives TTFT) ----
    if args.op_breakdown:
        from gllm_b200.utils.tracing import GraphTimer
        engine.prefill_timer = GraphTimer(eager=True)
    t_submit = time.perf_counter()
    ids = [engine.add_request(p, max_tokens=budget_tokens, temperature=0.0, eos_ids=[]) for p in prompts]
    first_token_at = {}
    guard = 0
    def prefilling():
        mine = 1 if engine.batcher.num_running < len(prompts) else 0
        if lockstep is None:
            return bool(mine)
        f = torch.tensor([mine], dtype=torch.int32, device=dev)      # lockstep engines step together until all are done
        dist.all_reduce(f, op=dist.ReduceOp.MAX)
        return bool(int(f[0]))

    while prefilling() and guard < 10000:
        engine.step()
        now = time.perf_counter()
        for rid, st in engine.reqs.items():
            if st.t_first > 0 and rid not in first_token_at:
                first_token_at[rid] = st.t_first - t_submit
        guard += 1
    ttft = sorted(first_token_at.values())
    prefill_s = time.perf_counter() - t_submit
    # ---- phase 2: warm-up decode steps through the public API (captures the graph) ----
    sampler = ClockSampler(local_rank)
    sampler.start()
    for _ in range(W + center_steps):
        engine.step()
    err = nv.device_error()
    if err:
        raise SystemExit(f"device error word {err} after warm-up")

    # ---- phase 3: e2e timed region: K engine steps incl. H2D of inputs and D2H of tokens ----
    sampler.lines.clear()      # the sampler has been running since before the warm-up; keep the timed regions' samples
    h2d0, d2h0 = engine.stats["h2d_bytes"], engine.stats["d2h_bytes"]
    tok0 = engine.stats["decode_tokens"]
    barrier()
    t0 = time.perf_counter()
    step_times = []
    for _ in range(K):
        ts = time.perf_counter()
        engine.step()
        step_times.append(time.perf_counter() - ts)
    torch.cuda.synchronize(dev)
    e2e_s = time.perf_counter() - t0
    e2e_tokens = engine.stats["decode_tokens"] - tok0
    h2d = (engine.stats["h2d_bytes"] - h2d0) / K
    d2h = (engine.stats["d2h_bytes"] - d2h0) / K

    # ---- phase 4: device-timed region: K replays of the captured decode step ----
    B = engine._bucket(args.concurrency)
    nv_calls0 = nv.CALLS[0]
    engine._decode_body(B) if args.no_graphs else None
    launches_per_step = (nv.CALLS[0] - nv_calls0) if args.no_graphs else engine.launches_per_graph.get(B, 0)
    graph = engine.graphs.get((B, True))
    run = (lambda: graph.replay()) if graph is not None else (lambda: engine._decode_body(B))
    for _ in range(3):
        run()
    barrier()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for _ in range(K):
        run()
    ev1.record()
    torch.cuda.synchronize(dev)
    dev_ms = ev0.elapsed_time(ev1)
    clocks = sampler.stop()
    err = nv.device_error()
    if err:
        raise SystemExit(f"device error word {err} in the timed region")

    # ---- phase 5 (N > 1): the baseline arm, same engine, same step, collectives on NCCL ----
    # unfused row-parallel GEMM -> ncclAllReduce -> residual/norm-statistics kernel, captured as its own CUDA graph
    nccl_ms = None
    if world > 1 and par == "tp" and tp is not None and tp.mode == "fused" and not args.no_baseline and graph is not None:
        tp.baseline = True
        keep = engine.graphs.pop((B, True))
        try:
            g2 = engine._capture(B)
            for _ in range(3):
                g2.replay()
            barrier()
            b0, b1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            b0.record()
            for _ in range(K):
                g2.replay()
            b1.record()
            torch.cuda.synchronize(dev)
            nccl_ms = b0.elapsed_time(b1)
        finally:
            tp.baseline = False
            engine.graphs[(B, True)] = keep
        err = nv.device_error()
        if err:
            raise SystemExit(f"device error word {err} in the baseline arm")

    prefill_ops = None
    if args.op_breakdown:
        prefill_ops = {n: round(v, 1) for n, v in engine.prefill_timer.results().items()}
        engine.prefill_timer = None
    breakdown = None
    if args.op_breakdown and not args.no_graphs:
        res = engine.decode_breakdown(B)
        names = sorted(res)
        bt = torch.tensor([res[n] for n in names], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(bt, op=dist.ReduceOp.MAX)
        breakdown = {n: round(float(v), 4) for n, v in zip(names, bt.tolist())}

    t = torch.tensor([dev_ms, e2e_s * 1e3, nccl_ms or 0.0], dtype=torch.float64, device=dev)
    cnt = torch.tensor([float(e2e_tokens)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        if ep_mode:
            dist.all_reduce(cnt, op=dist.ReduceOp.SUM)      # every rank served its own requests
    dev_ms, e2e_ms = float(t[0]), float(t[1])
    nccl_ms = float(t[2]) if nccl_ms is not None else None
    e2e_tokens = float(cnt[0])
    n_active = conc_total
    value = n_active * K / (dev_ms / 1e3)
    e2e_value = e2e_tokens / (e2e_ms / 1e3)
    if rank == 0:
        med = lambda xs: (sorted(xs)[len(xs) // 2] if xs else None)
        out = {
            "metric": "decode tokens/s", "value": round(value, 1), "unit": "tokens/s", "n_gpus": world, "steps": K,
            "warmup": W, "ms_per_step": round(dev_ms / K, 4), "higher_is_better": True, "scaling": "strong",
            "vs_baseline": (round(nccl_ms / dev_ms, 4) if nccl_ms else None), "dtype": "bf16", "data": "synthetic (random-init weights, uniform-random token ids)",
            "config": {"model": f"{args.model}-shape " + ("MoE decoder" if cfg.is_moe else "dense decoder"), "global_batch": n_active,
                       "seq_len": f"prompt U[{args.min_prompt},{args.max_prompt}] + {budget_tokens} out",
                       "parallelism": (f"ep{world} experts + data-parallel attention" if ep_mode else
                                       f"tp{tp_size}" + (f"pp{pp_size}" if pp_size > 1 else "")), "kv_page": 16, "shared_prefix": args.shared_prefix,
                       "l2": "inputs larger than L2: every step streams all weights and the KV cache",
                       "tp_form": getattr(tp, "form", "none"), "sequence_parallel": bool(getattr(model, "sequence_parallel", False)), "tp_mode": (getattr(tp, "mode", "none") + ("+multimem" if getattr(tp, "uses_multimem", False) else "")), "cuda_graphs": not args.no_graphs,
                       "layers": cfg.num_layers, "kv_dtype": args.kv_dtype,
                       "weight_quant": args.weight_quant, "expert_quant": args.expert_quant,
                       "valid": args.layers == 0 and (args.kv_dtype == "bf16" or args.model != "qwen3-8b")},
            "e2e": {"value": round(e2e_value, 1), "unit": "tokens/s", "h2d_bytes_per_step": int(h2d),
                    "d2h_bytes_per_step": int(d2h), "ms_per_step": round(e2e_ms / K, 4)},
            "gpu_launches": int(launches_per_step * K),
            "clocks": clocks,
            "p50_ttft_ms": round(med(ttft) * 1e3, 2) if ttft else None,
            "p50_tpot_ms": round(med(step_times) * 1e3, 4),
            "prefill_tokens_per_s": round(engine.stats["prefill_tokens"] / prefill_s, 1),
            "prefill_breakdown_ms": {"phase_wall": round(prefill_s * 1e3, 1),
                                     "prefill_calls_wall": round(engine.stats.get("prefill_wall_ms", 0.0), 1),
                                     "prefill_calls_device": round(engine.stats.get("prefill_device_ms", 0.0), 1),
                                     "prefill_steps": engine.stats["prefill_steps"]},
            "prefix_cache_hits": int(engine.batcher.prefix_hits) - prefix_hits0,
            "kv_pages": engine.num_pages,
        }
        if nccl_ms is not None:
            # the baseline arm: this engine with every collective on NCCL, measured in the same run
            out["baseline"] = {"what": "same engine, unfused row-parallel GEMM + ncclAllReduce + norm kernel (CUDA graph)",
                               "value": round(n_active * K / (nccl_ms / 1e3), 1), "unit": "tokens/s",
                               "ms_per_step": round(nccl_ms / K, 4)}
        if tp1_check is not None:
            # see phase 0: every chosen token within 0.25 standard deviations of the single-GPU maximum, and most of
            # them the exact single-GPU argmax
            out["config"]["tokens_match_tp1"] = (tp1_check["max_gap_sigma"] < 0.25 and
                                                 tp1_check["tokens_equal"] >= 0.6 * tp1_check["tokens_total"])
            out["config"]["tp1_check"] = tp1_check
        if breakdown is not None:
            out["decode_breakdown_ms"] = breakdown
        if prefill_ops is not None:
            out["prefill_ops_ms"] = prefill_ops
        print(json.dumps(out), flush=True)
    if world > 1:
        # Leave without tearing NCCL down: communicators referenced by captured CUDA graphs do not
        # destroy cleanly, and every rank has already contributed its numbers.
        dist.barrier()
        torch.cuda.synchronize(dev)
        sys.stdout.flush()
        os._exit(0)
    return 0


if __name__ == "__main__":
    sys.exit(main())
