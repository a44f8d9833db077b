"""Worker: a dense decoder with the residual stream sharded by rows (sequence parallel) against the same model with
all-reduce tensor parallelism and against the unsplit model. Argument: ``cpu`` (gloo ranks, fp32, the unfused
collectives) or a TPContext mode for CUDA ranks (``ll``, ``ll_p2p``, ``nccl``; bf16)."""
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
    from gllm_b200.engine.batch import ForwardBatch
    from gllm_b200.models.config import preset
    from gllm_b200.models.decoder import DecoderModel
    from gllm_b200.models.weights import RandomWeights
    from gllm_b200.parallel.tensor_parallel import TPContext
    cfg = preset("tiny-qwen3")
    cfg.hidden_size, cfg.num_heads, cfg.num_kv_heads, cfg.head_dim = 512, 4, 2, 128
    cfg.intermediate_size, cfg.num_layers, cfg.vocab_size = 768, 3, 1024
    dt = torch.float32 if cpu else torch.bfloat16
    src = RandomWeights(cfg, "cpu", torch.float32, seed=5, std=0.05)
    tp = TPContext(rank, world, dev, mode="nccl" if cpu else mode, max_tokens=256, hidden=cfg.hidden_size)
    if not cpu and mode != "nccl":
        assert tp.mode == "fused" and tp.form == "ll", getattr(tp, "setup_error", "")
    sp_model = DecoderModel(cfg, src, device=dev, dtype=dt, tp=tp, max_positions=256, sequence_parallel=True)
    ar_model = DecoderModel(cfg, src, device=dev, dtype=dt, tp=tp, max_positions=256)
    assert sp_model.sequence_parallel and sp_model.fused

    def i32(v):
        return torch.as_tensor(v, dtype=torch.int32, device=dev)

    def prefill(T):
        ids = (torch.arange(T, dtype=torch.int32) * 7 + 3) % cfg.vocab_size
        return ForwardBatch(token_ids=ids.to(dev), positions=i32(list(range(T))), slot_mapping=i32(list(range(T))),
                            block_tables=i32([list(range(8))]), ctx_lens=i32([T]), q_start=i32([0]), q_len=i32([T]),
                            max_q_len=T)

    def gathered(model, batch, kv):
        local = model.forward(batch, kv)[:, :model.vocab_local].float().contiguous()
        parts = [torch.empty_like(local) for _ in range(world)]
        dist.all_gather(parts, local)
        return torch.cat(parts, 1).cpu()

    tol = dict(rtol=1e-3, atol=2e-4) if cpu else dict(rtol=0.05, atol=0.05)
    for T in (37, 128, 5, 1):      # odd row counts: the last rank owns fewer rows (or none)
        kv_sp, kv_ar = sp_model.alloc_kv_cache(8), ar_model.alloc_kv_cache(8)
        got = gathered(sp_model, prefill(T), kv_sp)
        want = gathered(ar_model, prefill(T), kv_ar)
        torch.testing.assert_close(got, want, **tol)
        for a, b in zip(kv_sp, kv_ar):      # the same keys and values reach the cache
            torch.testing.assert_close(a.float().cpu(), b.float().cpu(), **tol)
        if rank == 0 and cpu:
            ref = DecoderModel(cfg, src, device="cpu", dtype=dt, max_positions=256)
            full = ref.forward(prefill(T), ref.alloc_kv_cache(8))[:, :cfg.vocab_size]
            torch.testing.assert_close(got, full.float(), **tol)
    if not cpu:
        from gllm_b200.ops import _native as nv
        torch.cuda.synchronize()
        assert nv.device_error() == 0
    dist.barrier()
    print("SP_DECODER_WORKER_OK", rank, mode, flush=True)
    tp.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
