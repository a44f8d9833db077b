"""Worker: one sequence-parallel block over row-sharded activations (all-gather in front of a column-parallel GEMM,
reduce-scatter behind the row-parallel GEMM), compared with the fp32 product of the unsharded operands.
Argument: ``cpu`` (gloo ranks, the unfused fall-backs) or a TPContext mode for CUDA ranks (``ll``, ``ll_p2p``, ``nccl``)."""
import os
import sys

import torch
import torch.distributed as dist


def main():
    mode = sys.argv[1] if len(sys.argv) > 1 else "cpu"
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    cpu = mode == "cpu"
    if cpu:
        dev = torch.device("cpu")
        dist.init_process_group("gloo")
    else:
        torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
        dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
        dist.init_process_group("nccl", device_id=dev)
    from gllm_b200 import ops
    from gllm_b200.parallel.tensor_parallel import TPContext
    H, I = 512, 768                       # hidden size, intermediate size of the whole layer (divisible by 2, 3, 4)
    tp = TPContext(rank, world, dev, mode="nccl" if cpu else mode, max_tokens=256, hidden=H)
    if not cpu and mode != "nccl":
        assert tp.mode == "fused" and tp.form == "ll", getattr(tp, "setup_error", "")
    g = torch.Generator().manual_seed(11)
    dt = torch.bfloat16
    for it, M in enumerate([256, 77, 256, 130]):
        x_full = torch.randn(M, H, generator=g).to(dt)
        w_up = (torch.randn(I, H, generator=g) * 0.05).to(dt)          # column-parallel: rows split over ranks
        w_down = (torch.randn(H, I, generator=g) * 0.05).to(dt)        # row-parallel: columns split over ranks
        ref_mid = (x_full.float() @ w_up.float().t()).to(dt).float()
        ref_out = ref_mid @ w_down.float().t() + x_full.float()
        lo, n_own = tp.shard_rows(M)
        per = (M + world - 1) // world
        Il = I // world
        x_shard = torch.zeros(per, H, dtype=dt, device=dev)
        x_shard[:n_own].copy_(x_full[lo:lo + n_own])
        wu = w_up[rank * Il:(rank + 1) * Il].contiguous().to(dev)
        wd = w_down[:, rank * Il:(rank + 1) * Il].contiguous().to(dev)
        # all-gather + column-parallel GEMM: every rank gets all M rows of its Il columns
        a_full = torch.zeros(M, H, dtype=dt, device=dev)
        tp.allgather_input(x_shard, a_full)
        mid = ops.gemm(a_full, wu, bn=128)
        if not cpu:
            torch.cuda.synchronize()
        assert torch.equal(a_full.cpu(), x_full), f"rank {rank} iter {it}: gathered rows differ"
        err = (mid.float().cpu() - ref_mid[:, rank * Il:(rank + 1) * Il]).abs().max().item()
        assert err < 0.05 * ref_mid.abs().max().item(), f"rank {rank} iter {it}: column-parallel err {err}"
        # row-parallel GEMM + reduce-scatter: the rank keeps its rows of the sum, added to its residual shard
        ss = torch.zeros(per, (H + 255) // 256, device=dev)
        res = x_shard.clone()
        tp.gemm_reduce_scatter_residual(mid, wd, res, ss, M)
        if not cpu:
            torch.cuda.synchronize()
        want = ref_out[lo:lo + n_own]
        row_err = (res[:n_own].float().cpu() - want).abs().amax(-1) if n_own else torch.zeros(0)
        bad = (row_err > 0.03 * want.abs().amax(-1) + 0.05).nonzero().flatten() if n_own else row_err
        assert bad.numel() == 0, f"rank {rank} iter {it}: rows {bad[:8].tolist()} off by {row_err[bad[:8]].tolist()}"
        if n_own:
            torch.testing.assert_close(ss[:n_own].sum(-1).cpu(), res[:n_own].float().pow(2).sum(-1).cpu(), rtol=3e-3, atol=3e-3)
    if not cpu:
        from gllm_b200.ops import _native as nv
        assert nv.device_error() == 0
    dist.barrier()
    print("SP_WORKER_OK", rank, mode, tp.form, flush=True)
    tp.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
