"""Worker for the expert-parallel tests (torchrun, one rank per process). ``gloo`` on CPU checks the all-to-all
transport; ``nccl`` on GPUs checks the fused peer-memory transport against the same fp32 oracle."""
import os
import sys
from types import SimpleNamespace

import torch
import torch.distributed as dist


def main():
    mode = sys.argv[1] if len(sys.argv) > 1 else "a2a"
    on_gpu = mode != "cpu"
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    if on_gpu:
        torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
        dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
        dist.init_process_group("nccl", device_id=dev)
        dtype = torch.bfloat16
    else:
        dev = torch.device("cpu")
        dist.init_process_group("gloo")
        dtype = torch.float32
    from gllm_b200.models.config import preset
    from gllm_b200.models.moe import pack_moe_layer
    from gllm_b200.models.weights import RandomWeights
    from gllm_b200.parallel.expert_parallel import EPContext

    cfg = preset("tiny-moe")
    cfg.num_experts, cfg.num_experts_per_tok, cfg.num_shared_experts = 8, 2, 1
    src = RandomWeights(cfg, "cpu", torch.float32, seed=5, std=0.08)
    H = cfg.hidden_size
    ep = EPContext(rank, world, dev, num_experts=cfg.num_experts, hidden=H, top_k=cfg.num_experts_per_tok,
                   max_tokens=320, mode={"cpu": "a2a", "a2a": "a2a", "fused": "fused"}[mode])
    assert ep.mode == ("fused" if mode == "fused" else "a2a"), getattr(ep, "setup_error", "")
    fused_model = on_gpu
    layer = pack_moe_layer(cfg, src, 0, 0, 1, dev, dtype, ep=ep, fused=fused_model)
    oracle = pack_moe_layer(cfg, src, 0, 0, 1, torch.device("cpu"), torch.float32, ep=None, fused=False)
    post = src.get("L0.post_attn_norm").float()
    model = SimpleNamespace(act_id=0, device=dev, dtype=dtype)
    cpu_model = SimpleNamespace(act_id=0, device=torch.device("cpu"), dtype=torch.float32)
    g = torch.Generator().manual_seed(100 + rank)
    worst = 0.0
    for it, T in enumerate([37 + 11 * rank, 1, 300 - 40 * rank, 0 if rank == 1 else 5, 64]):
        x0 = torch.randn(T, H, generator=g)
        if dtype == torch.bfloat16:
            x0 = x0.to(torch.bfloat16).float()
        # oracle: normalise, full expert set, add into the residual
        var = x0.pow(2).mean(-1, keepdim=True)
        h = x0 * torch.rsqrt(var + cfg.rms_norm_eps) * post
        want = x0.clone()
        if T > 0:
            oracle.forward_unfused(cpu_model, want, h, T)
        x = x0.clone().to(dev, dtype).contiguous()
        if fused_model:
            ss_in = x.float().pow(2).sum(-1, keepdim=True).contiguous()
            ss_out = torch.zeros(max(T, 1), 1, device=dev)
            Tq = T
            if T == 0:  # the kernels still run (this rank's experts serve the others) with an empty token list
                x = torch.zeros(1, H, device=dev, dtype=dtype)
                ss_in = torch.ones(1, 1, device=dev)
            ws = layer.workspace(model, max(T, 1))
            ids, w = layer._route(x[:max(T, 1)], ss_in, ws, max(T, 1), H, cfg.rms_norm_eps)
            ep.moe_forward(layer, model, x, ss_in, ss_out, ids[:Tq], w[:Tq], ws, Tq)
            torch.cuda.synchronize()
            if T > 0:
                torch.testing.assert_close(ss_out[:T, 0].cpu(), x[:T].float().pow(2).sum(-1).cpu(), rtol=3e-3, atol=3e-3)
        else:
            hh = h.to(dev, dtype)
            if T == 0:
                ids = torch.zeros((0, cfg.num_experts_per_tok), dtype=torch.int32, device=dev)
                w = torch.zeros((0, cfg.num_experts_per_tok), dtype=torch.float32, device=dev)
                ep.moe_forward(layer, model, x, None, None, ids, w, None, 0, normalised_input=hh)
            else:
                layer.forward_unfused(model, x, hh, T)
        if T > 0:
            got = x[:T].float().cpu()
            err = (got - want).abs().max().item()
            scale = (want - x0).abs().max().item() + 1e-6
            worst = max(worst, err / scale)
            tol = 0.06 if dtype == torch.bfloat16 else 1e-4
            assert err <= tol * max(scale, 1.0), f"rank {rank} iter {it} T {T} err {err} scale {scale}"
    if on_gpu:
        from gllm_b200.ops import _native as nv
        code = nv.device_error()
        assert code == 0, f"device error {code}"
    dist.barrier()
    print("EP_WORKER_OK", mode, rank, f"worst_rel={worst:.4f}", flush=True)
    if on_gpu:
        os._exit(0)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
