"""Worker for the multi-GPU test of the block-scaled row-parallel GEMM with the fused all-reduce (launched by
torchrun, one rank per GPU). Arguments: TPContext mode (``ll`` / ``ll_p2p``) and operand format (``mxfp8`` / ``nvfp4``)."""
import os
import sys

import torch
import torch.distributed as dist


def main():
    mode, fmt = sys.argv[1], sys.argv[2]
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl", device_id=dev)
    from gllm_b200.ops import _native as nv
    from gllm_b200.ops import blockscale as B
    from gllm_b200.parallel.tensor_parallel import TPContext
    H = 2048
    tp = TPContext(rank, world, dev, mode=mode, max_tokens=2048, hidden=H)
    assert tp.mode == "fused" and tp.form == "ll", getattr(tp, "setup_error", "")
    g = torch.Generator(device="cpu").manual_seed(9)
    for it, (M, K) in enumerate([(256, 1024), (77, 512), (256, 2048), (1500, 1024), (64, 4096), (256, 1024)]):
        a_full = torch.randn(M, K * world, generator=g).to(torch.bfloat16)
        w_full = (torch.randn(H, K * world, generator=g) * 0.05).to(torch.bfloat16)
        x0 = torch.randn(M, H, generator=g).to(torch.bfloat16).to(dev)
        w = B.quantize(w_full[:, rank * K:(rank + 1) * K].contiguous(), fmt).to(dev)
        a = a_full[:, rank * K:(rank + 1) * K].contiguous().to(dev)
        aq = B.quantize_act(a, fmt, tensor_scale=1.0 / 64.0) if fmt == "nvfp4" else B.quantize_act(a, fmt)
        ref = aq.dequantize()[:M].float() @ w.dequantize().float().t()
        dist.all_reduce(ref)
        ref = ref + x0.float()
        assert tp.can_fuse_blockscaled(M, H)
        x = x0.clone()
        ss = tp.gemm_allreduce_residual_bs(aq, w, x, torch.zeros(M, H // 128, device=dev))
        torch.cuda.synchronize()
        row_err = (x.float() - ref).abs().amax(-1)
        bad = (row_err > 0.03 * ref.abs().amax(-1) + 0.05).nonzero().flatten()
        assert bad.numel() == 0, f"rank {rank} iter {it} {fmt}: rows {bad[:8].tolist()} off by {row_err[bad[:8]].tolist()}"
        torch.testing.assert_close(ss.sum(-1), x.float().pow(2).sum(-1), rtol=2e-3, atol=2e-3)
        # every rank holds the same rows
        mine = x.float().contiguous()
        other = mine.clone()
        dist.broadcast(other, src=0)
        assert torch.equal(mine, other), f"rank {rank} iter {it}: rows differ between ranks"
    assert nv.device_error() == 0
    dist.barrier()
    if rank == 0:
        print("TP_BS_WORKER_OK", mode, fmt, "multimem" if tp.uses_multimem else "p2p", flush=True)
    tp.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
