"""Times one expert-parallel MoE layer (route -> dispatch -> expert GEMMs -> combine) per transport.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        -m gllm_b200.parallel.ep_bench [--tokens 256] [--hidden 2048] [--experts 128] [--topk 8] [--inter 768]

Defaults are the Qwen3-30B-A3B layer shape. Each rank routes ``tokens`` rows of its own. Reported times are
CUDA-event times of a CUDA-graph replay of ``layers`` back-to-back layer calls, maximum over ranks, per layer.
"""
from __future__ import annotations

import argparse
import json
import os
from types import SimpleNamespace

import torch
import torch.distributed as dist


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=256)
    ap.add_argument("--hidden", type=int, default=2048)
    ap.add_argument("--experts", type=int, default=128)
    ap.add_argument("--topk", type=int, default=8)
    ap.add_argument("--inter", type=int, default=768)
    ap.add_argument("--layers", type=int, default=8)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--modes", default="fused,a2a")
    a = ap.parse_args()
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    from ..models.config import ModelConfig
    from ..models.moe import pack_moe_layer
    from ..models.weights import RandomWeights
    from .expert_parallel import EPContext
    cfg = ModelConfig(arch="qwen3_moe", hidden_size=a.hidden, num_layers=1, num_heads=16, num_kv_heads=4, head_dim=128,
                      intermediate_size=a.inter, vocab_size=1024, num_experts=a.experts, num_experts_per_tok=a.topk,
                      moe_intermediate_size=a.inter)
    src = RandomWeights(cfg, dev, torch.bfloat16, seed=1, std=0.03)
    model = SimpleNamespace(act_id=0, device=dev, dtype=torch.bfloat16)
    T, H = a.tokens, a.hidden
    out = {"world": world, "tokens_per_rank": T, "hidden": H, "experts": a.experts, "topk": a.topk, "inter": a.inter}
    for mode in a.modes.split(","):
        ep = EPContext(rank, world, dev, num_experts=a.experts, hidden=H, top_k=a.topk, max_tokens=T, mode=mode)
        layer = pack_moe_layer(cfg, src, 0, 0, 1, dev, torch.bfloat16, ep=ep, fused=True)
        x = torch.randn(T, H, device=dev).to(torch.bfloat16)
        ss_in = x.float().pow(2).sum(-1, keepdim=True).contiguous()
        ss_out = torch.zeros(T, 1, device=dev)
        assert a.layers % 2 == 0

        def run_layers():
            # the statistics of one layer's output feed the next layer's norm, as in the decoder
            for i in range(a.layers):
                layer.forward(model, x, ss_in if i % 2 == 0 else ss_out, ss_out if i % 2 == 0 else ss_in, T)

        for _ in range(3):
            run_layers()
        torch.cuda.synchronize()
        dist.barrier()
        graph = None
        if mode == "fused":   # the all-to-all transport reads split sizes on the host: not capturable
            side = torch.cuda.Stream()
            with torch.cuda.stream(side):
                run_layers()
                torch.cuda.synchronize()
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=side):
                    run_layers()
            torch.cuda.synchronize()
        times = []
        for it in range(a.iters):
            x.copy_(torch.randn(T, H, device=dev).to(torch.bfloat16))
            ss_in.copy_(x.float().pow(2).sum(-1, keepdim=True))
            dist.barrier()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            graph.replay() if graph is not None else run_layers()
            e1.record()
            torch.cuda.synchronize()
            times.append(e0.elapsed_time(e1) * 1e3 / a.layers)
        t = torch.tensor(sorted(times)[len(times) // 2], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        out[f"{mode}_us_per_layer"] = round(float(t), 2)
        from ..ops import _native as nv
        out[f"{mode}_device_error"] = nv.device_error()
        ep.close()
    # bytes a rank sends per layer: T*k rows out and back
    out["nvlink_bytes_per_rank_per_layer"] = 2 * T * a.topk * H * 2 * (world - 1) // max(world, 1)
    if rank == 0:
        print(json.dumps(out), flush=True)
    dist.barrier()
    os._exit(0)


if __name__ == "__main__":
    main()
