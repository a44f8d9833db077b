"""Worker: serving engines in lockstep, data-parallel attention + expert-parallel MoE (torchrun; gloo on CPU with the
all-to-all transport, nccl on GPUs with the fused peer-memory transport). Every rank serves its OWN requests."""
import os
import sys

import torch
import torch.distributed as dist


def main():
    mode = sys.argv[1] if len(sys.argv) > 1 else "cpu"
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    if mode == "cpu":
        dist.init_process_group("gloo")
        dev, dtype, ep_mode = torch.device("cpu"), torch.float32, "a2a"
    else:
        torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
        dev, dtype, ep_mode = torch.device("cuda", int(os.environ["LOCAL_RANK"])), torch.bfloat16, "fused"
        dist.init_process_group("nccl", device_id=dev)
    from gllm_b200.engine.executor import EngineConfig, LLMEngine
    from gllm_b200.models.config import preset
    from gllm_b200.models.decoder import DecoderModel
    from gllm_b200.models.weights import RandomWeights
    from gllm_b200.parallel.expert_parallel import EPContext
    cfg = preset("tiny-moe")
    src = RandomWeights(cfg, "cpu", torch.float32, seed=2, std=0.05)
    ep = EPContext(rank, world, dev, num_experts=cfg.num_experts, hidden=cfg.hidden_size, top_k=cfg.num_experts_per_tok,
                   max_tokens=128, mode=ep_mode)
    model = DecoderModel(cfg, src, device=dev, dtype=dtype, max_positions=256, ep=ep)
    assert model.layers[0].moe.ep is ep and model.layers[0].moe.e_local == cfg.num_experts // world
    ec = EngineConfig(max_num_seqs=4, max_model_len=128, max_batch_tokens=64, prefill_chunk=48, num_pages=64)
    eng = LLMEngine(model, ec, lockstep_group=dist.group.WORLD)
    eng.precapture()
    # different work per rank: counts, prompt lengths and output lengths all differ, so ranks idle at different times
    prompts = [[(7 * i + 3 * rank + j) % cfg.vocab_size for j in range(5 + 9 * i + 20 * rank)] for i in range(2 + rank)]
    max_new = [4 + 3 * i + 5 * (1 - rank) for i in range(len(prompts))]
    ids = [eng.submit(p, max_tokens=m, temperature=0.0, eos_ids=[]) for p, m in zip(prompts, max_new)]
    eng.run_until_done()
    got = [eng.results[i].token_ids for i in ids]
    # oracle: the unsplit model in an ordinary engine (CPU fp32)
    ref_model = DecoderModel(cfg, src, device="cpu", dtype=torch.float32, max_positions=256)
    ref = LLMEngine(ref_model, EngineConfig(max_num_seqs=4, max_model_len=128, max_batch_tokens=64, prefill_chunk=48, num_pages=64))
    rids = [ref.submit(p, max_tokens=m, temperature=0.0, eos_ids=[]) for p, m in zip(prompts, max_new)]
    ref.run_until_done()
    want = [ref.results[i].token_ids for i in rids]
    for g, w in zip(got, want):
        assert len(g) == len(w)
        if mode == "cpu":
            assert g == w, (g, w)
        else:
            assert g[:2] == w[:2], (g, w)      # bf16 may diverge late
    dist.barrier()
    print("EP_ENGINE_WORKER_OK", rank, [len(g) for g in got], flush=True)
    if mode != "cpu":
        os._exit(0)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
