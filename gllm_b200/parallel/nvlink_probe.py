"""NVLink bytes per launch of the fused multi-GPU kernels, by difference of the GPU's own (read-only) NVML counters.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        -m gllm_b200.parallel.nvlink_probe [--what ar,ep] [--replays 1000] [--tp-mode ll|fused|pull]

A kernel that waits for another rank cannot sit under a profiler (its replay passes would run on one rank only), so the
evidence for the bytes it moves is the difference of ``NVML_FI_DEV_NVLINK_THROUGHPUT_DATA_TX / RX`` (KiB, summed over
the links of the GPU) before and after a loop of CUDA-graph replays, divided by the number of launches, set beside
the algorithmic bytes:

* row-parallel GEMM + all-reduce, ownership forms (``ll`` / ``fused``): a rank sends (W-1)/W of its [M, N] bf16 partial
  to the row owners and (W-1) copies of its M/W finished rows: 2 * (W-1)/W * M * N * 2 bytes out, the same in;
  ``pull`` one-shot: every rank reads (W-1) partials: (W-1) * M * N * 2 bytes in.
* one expert-parallel MoE layer: each routed row leaves and comes back: 2 * T * k * H * 2 * (W-1)/W bytes.

Nothing here changes a GPU setting: the counters are only read.
"""
from __future__ import annotations

import argparse
import json
import os
from types import SimpleNamespace

import torch
import torch.distributed as dist

_TX, _RX = 138, 139      # NVML_FI_DEV_NVLINK_THROUGHPUT_DATA_TX / _RX (KiB since the driver loaded)


LAST_NVML_STATUS = "ok"


def read_nvlink_kib(handle):
    """(tx_kib, rx_kib) summed over all links (scope id 0xFFFFFFFF), or None when the driver does not report them
    (``LAST_NVML_STATUS`` then says what NVML answered)."""
    global LAST_NVML_STATUS
    import pynvml
    try:
        vals = pynvml.nvmlDeviceGetFieldValues(handle, [(_TX, 0xFFFFFFFF), (_RX, 0xFFFFFFFF)])
    except pynvml.NVMLError as exc:
        LAST_NVML_STATUS = f"nvmlDeviceGetFieldValues raised {exc!r}"
        return None
    out = []
    for v in vals:
        if v.nvmlReturn != 0:
            LAST_NVML_STATUS = f"field {getattr(v, 'fieldId', '?')}: nvmlReturn {v.nvmlReturn}"
            return None
        out.append(int(v.value.ullVal))
    LAST_NVML_STATUS = "ok"
    return tuple(out)


def _nvml_handle(local_rank: int):
    import pynvml
    pynvml.nvmlInit()
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    idx = int(vis.split(",")[local_rank]) if vis and vis.split(",")[local_rank].isdigit() else local_rank
    return pynvml.nvmlDeviceGetHandleByIndex(idx)


def _measure(handle, graph, replays, dev):
    dist.barrier()
    torch.cuda.synchronize(dev)
    before = read_nvlink_kib(handle)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(replays):
        graph.replay()
    e1.record()
    torch.cuda.synchronize(dev)
    dist.barrier()
    after = read_nvlink_kib(handle)
    ms = e0.elapsed_time(e1)
    if before is None or after is None:
        return None, None, ms
    return (after[0] - before[0]) * 1024, (after[1] - before[1]) * 1024, ms


def _capture(fn, dev):
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        for _ in range(3):
            fn()
        torch.cuda.synchronize(dev)
        dist.barrier()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=side):
            fn()
    torch.cuda.synchronize(dev)
    return g


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--what", default="ar,ep")
    ap.add_argument("--replays", type=int, default=1000)
    ap.add_argument("--tp-mode", default="ll")
    ap.add_argument("--m", type=int, default=256)
    ap.add_argument("--n", type=int, default=4096)
    ap.add_argument("--k", type=int, default=4096, help="K of the whole GEMM; each rank multiplies K / world")
    a = ap.parse_args()
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    handle = _nvml_handle(local)
    from ..ops import _native as nv
    out = {"world": world, "replays": a.replays, "counters": "NVML_FI_DEV_NVLINK_THROUGHPUT_DATA_TX/RX"}
    per_graph = 8        # launches per captured graph

    if "ar" in a.what.split(","):
        from .tensor_parallel import TPContext
        M, N, K = a.m, a.n, a.k // world
        tp = TPContext(rank, world, dev, mode=a.tp_mode, max_tokens=max(M, 256), hidden=N)
        x = torch.randn(M, N, device=dev).to(torch.bfloat16)
        act = torch.randn(M, K, device=dev).to(torch.bfloat16)
        ws = [(torch.randn(N, K, device=dev) * 0.02).to(torch.bfloat16) for _ in range(per_graph)]
        ss = torch.zeros(M, N // 256, device=dev)      # the fused kernels report statistics per 256 columns
        part = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
        bufs = tp.workspace_buffers(M) if tp.form == "push" else None
        if bufs is not None:
            bufs["x"].copy_(x)
            x = bufs["x"]

        def run():
            for w in ws:
                tp.gemm_allreduce_residual(act, w, x, ss, part)
                x.mul_(0.5)       # keeps the residual stream bounded over thousands of launches

        g = _capture(run, dev)
        tx, rx, ms = _measure(handle, g, a.replays // per_graph, dev)
        launches = (a.replays // per_graph) * per_graph
        if tp.form in ("ll", "push"):
            algo = 2 * (world - 1) * M * N * 2 // world
        else:
            algo = (world - 1) * M * N * 2
        res = {"shape": [M, N, K], "form": tp.form, "multimem": tp.uses_multimem, "launches": launches,
               "us_per_launch": round(ms * 1e3 / launches, 2), "algorithmic_bytes_per_launch": algo}
        if tx is not None:
            res.update(tx_bytes_per_launch=tx // launches, rx_bytes_per_launch=rx // launches,
                       tx_over_algorithmic=round(tx / launches / algo, 3), rx_over_algorithmic=round(rx / launches / algo, 3))
        else:
            res["counters_unavailable"] = LAST_NVML_STATUS
        res["device_error"] = nv.device_error()
        out["gemm_allreduce"] = res
        tp.close()

    if "ep" in a.what.split(","):
        from ..models.config import ModelConfig
        from ..models.moe import pack_moe_layer
        from ..models.weights import RandomWeights
        from .expert_parallel import EPContext
        T, H, E, k, inter = 256, 2048, 128, 8, 768
        cfg = ModelConfig(arch="qwen3_moe", hidden_size=H, num_layers=1, num_heads=16, num_kv_heads=4, head_dim=128,
                          intermediate_size=inter, vocab_size=1024, num_experts=E, num_experts_per_tok=k,
                          moe_intermediate_size=inter)
        src = RandomWeights(cfg, dev, torch.bfloat16, seed=1, std=0.03)
        model = SimpleNamespace(act_id=0, device=dev, dtype=torch.bfloat16)
        ep = EPContext(rank, world, dev, num_experts=E, hidden=H, top_k=k, max_tokens=T, mode="fused")
        layer = pack_moe_layer(cfg, src, 0, 0, 1, dev, torch.bfloat16, ep=ep, fused=True)
        x = torch.randn(T, H, device=dev).to(torch.bfloat16)
        ss_a = x.float().pow(2).sum(-1, keepdim=True).contiguous()
        ss_b = torch.zeros(T, 1, device=dev)

        def run_ep():
            for i in range(per_graph):
                layer.forward(model, x, ss_a if i % 2 == 0 else ss_b, ss_b if i % 2 == 0 else ss_a, T)
                x.mul_(0.5)

        g = _capture(run_ep, dev)
        tx, rx, ms = _measure(handle, g, a.replays // per_graph, dev)
        launches = (a.replays // per_graph) * per_graph
        algo = 2 * T * k * H * 2 * (world - 1) // world
        res = {"tokens_per_rank": T, "hidden": H, "experts": E, "topk": k, "layers": launches,
               "us_per_layer": round(ms * 1e3 / launches, 2), "algorithmic_bytes_per_layer": algo}
        if tx is not None:
            res.update(tx_bytes_per_layer=tx // launches, rx_bytes_per_layer=rx // launches,
                       tx_over_algorithmic=round(tx / launches / algo, 3))
        else:
            res["counters_unavailable"] = LAST_NVML_STATUS
        res["device_error"] = nv.device_error()
        out["ep_layer"] = res
        ep.close()

    gathered = [None] * world
    dist.all_gather_object(gathered, out)
    if rank == 0:
        print(json.dumps({"rank0": out, "tx_all_ranks": [
            {k2: v.get("tx_bytes_per_launch", v.get("tx_bytes_per_layer")) for k2, v in o.items() if isinstance(v, dict)}
            for o in gathered]}), flush=True)
    dist.barrier()
    os._exit(0)


if __name__ == "__main__":
    main()
