"""Worker: tensor-parallel attention + expert-parallel FFN on the same ranks (torchrun; gloo on CPU, nccl on GPUs).
Every rank runs the same batch; the vocabulary-sharded logits are gathered and compared with the unsplit model."""
import os
import sys

import torch
import torch.distributed as dist


def main():
    mode = sys.argv[1] if len(sys.argv) > 1 else "cpu"
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    if mode == "cpu":
        dist.init_process_group("gloo")
        dev, dtype = torch.device("cpu"), torch.float32
    else:
        torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
        dev, dtype = torch.device("cuda", int(os.environ["LOCAL_RANK"])), torch.bfloat16
        dist.init_process_group("nccl", device_id=dev)
    from gllm_b200.engine.batch import ForwardBatch
    from gllm_b200.models.config import preset
    from gllm_b200.models.decoder import DecoderModel
    from gllm_b200.models.weights import RandomWeights
    from gllm_b200.parallel.tensor_parallel import TPContext
    cfg = preset("tiny-moe")
    cfg.num_shared_experts = 1
    src = RandomWeights(cfg, "cpu", torch.float32, seed=2, std=0.05)
    tp = TPContext(rank, world, dev, mode="nccl" if mode == "cpu" else "auto", max_tokens=256, hidden=cfg.hidden_size)
    model = DecoderModel(cfg, src, device=dev, dtype=dtype, tp=tp, max_positions=256)
    assert model.layers[0].moe.tp_experts is tp and model.layers[0].moe.e_local == cfg.num_experts // world
    T = 45
    ids = (torch.arange(T, dtype=torch.int32) * 7 + 3) % cfg.vocab_size

    def batch(d):
        return ForwardBatch(token_ids=ids.to(d), positions=torch.arange(T, dtype=torch.int32, device=d),
                            slot_mapping=torch.arange(T, dtype=torch.int32, device=d),
                            block_tables=torch.arange(8, dtype=torch.int32, device=d)[None],
                            ctx_lens=torch.tensor([T], dtype=torch.int32, device=d),
                            q_start=torch.tensor([0], dtype=torch.int32, device=d),
                            q_len=torch.tensor([T], dtype=torch.int32, device=d), max_q_len=T)
    local = model.forward(batch(dev), model.alloc_kv_cache(8))[:, :model.vocab_local].float().contiguous()
    parts = [torch.empty_like(local) for _ in range(world)]
    dist.all_gather(parts, local)
    got = torch.cat(parts, 1).cpu()
    if rank == 0:
        ref = DecoderModel(cfg, src, device="cpu", dtype=torch.float32, max_positions=256)
        want = ref.forward(batch("cpu"), ref.alloc_kv_cache(8))[:, :cfg.vocab_size]
        cos = torch.nn.functional.cosine_similarity(got.flatten(), want.flatten(), dim=0).item()
        assert cos > (0.9999 if mode == "cpu" else 0.995), cos
        if mode == "cpu":
            torch.testing.assert_close(got, want, rtol=1e-3, atol=1e-4)
    if mode == "cpu":      # validated with gloo ranks; the GPU run of this worker keeps to the kernels it was measured with
        # load balancing: mirror two hot experts on every rank (one owned by each rank when world == 2); the logits stay
        # what they were, the rows of those experts are now shared out over the ranks
        hot = [1, cfg.num_experts - 1]
        for lw in model.layers:
            if lw.moe is not None:
                lw.moe.set_mirrors(hot, model)
        again = model.forward(batch(dev), model.alloc_kv_cache(8))[:, :model.vocab_local].float().contiguous()
        torch.testing.assert_close(again, local, rtol=1e-3 if mode == "cpu" else 0.05, atol=1e-4 if mode == "cpu" else 0.05)
        moe0 = next(lw.moe for lw in model.layers if lw.moe is not None)
        assert moe0.n_mirror == 2 and moe0.mirrored == (1, cfg.num_experts - 1)
        for lw in model.layers:
            if lw.moe is not None:
                lw.moe.set_mirrors([], model)
        back = model.forward(batch(dev), model.alloc_kv_cache(8))[:, :model.vocab_local].float().contiguous()
        torch.testing.assert_close(back, local, rtol=1e-3 if mode == "cpu" else 0.05, atol=1e-4 if mode == "cpu" else 0.05)
        # the engine's load balancer: a skewed window names expert 2 hot, every rank mirrors it, the tokens do not change
        from gllm_b200.engine.executor import EngineConfig, LLMEngine
        eng = LLMEngine(model, EngineConfig(max_num_seqs=2, max_model_len=128, max_batch_tokens=64, prefill_chunk=64, num_pages=32,
                                            use_cuda_graphs=False))
        prompts = [ids[:20].tolist(), ids[5:30].tolist()]
        before = [r.token_ids for r in eng.generate_batch(prompts, max_tokens=5, temperature=0.0, eos_ids=[])]
        obs = eng.coordinators.observability
        assert obs.eplb is not None
        skew = torch.ones(cfg.num_experts, dtype=torch.int64)
        skew[2] = 50 * cfg.num_experts
        obs.eplb.samples.clear()
        obs.eplb.record(skew)
        assert eng.rebalance_experts(reduce=True) == [2] and moe0.mirrored == (2,) and eng.stats["expert_rebalances"] == 1
        after = [r.token_ids for r in eng.generate_batch(prompts, max_tokens=5, temperature=0.0, eos_ids=[])]
        assert after == before
    dist.barrier()
    print("TP_MOE_WORKER_OK", rank, flush=True)
    if mode != "cpu":
        os._exit(0)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
