"""Worker (gloo ranks): a long prompt prefilled by the engines of all ranks together, then decoded by each."""
import os

import torch
import torch.distributed as dist


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo")
    from gllm_b200.engine.executor import EngineConfig, LLMEngine
    from gllm_b200.models.config import preset
    from gllm_b200.models.decoder import DecoderModel
    from gllm_b200.models.weights import RandomWeights
    cfg = preset("tiny-qwen3")
    src = RandomWeights(cfg, "cpu", torch.float32, seed=4, std=0.05)
    model = DecoderModel(cfg, src, device="cpu", dtype=torch.float32, max_positions=256)
    ecfg = dict(max_num_seqs=2, max_model_len=200, max_batch_tokens=128, prefill_chunk=128, num_pages=40 + rank)
    prompt = ((torch.arange(103) * 11 + 5) % cfg.vocab_size).tolist()          # 6 full pages + 7 tokens
    eng = LLMEngine(model, EngineConfig(**ecfg))
    if rank == 1:      # a different pool state on this rank: the logical pages land under other page ids
        eng.generate_batch([[9, 8, 7] * 12], max_tokens=2, temperature=0.0, eos_ids=[])
    rid = eng.add_request_context_parallel(prompt, rank, world, max_tokens=6, temperature=0.0, eos_ids=[])
    eng.run_until_done()
    res = eng.results[rid]
    per = -(-6 // world) * 16
    assert eng.stats["cp_prefills"] == 1 and eng.stats["cp_prefill_tokens"] == min(96, (rank + 1) * per) - rank * per
    assert res.telemetry.cached_prefix_tokens == 96, res.telemetry
    everyone = [None] * world
    dist.all_gather_object(everyone, res.token_ids)
    assert all(t == everyone[0] for t in everyone)
    if rank == 0:
        one = LLMEngine(model, EngineConfig(**ecfg))
        want = one.generate_batch([prompt], max_tokens=6, temperature=0.0, eos_ids=[])[0].token_ids
        assert res.token_ids == want, (res.token_ids, want)
    # a prompt long enough for two chunks per rank: zig-zag shards (balanced causal work)
    if world == 2:
        long2 = ((torch.arange(140) * 13 + 1) % cfg.vocab_size).tolist()      # 8 full pages + 12 tokens
        rid3 = eng.add_request_context_parallel(long2, rank, world, max_tokens=4, temperature=0.0, eos_ids=[])
        eng.run_until_done()
        assert eng.stats["cp_prefills"] == 2 and eng.results[rid3].telemetry.cached_prefix_tokens == 128
        if rank == 0:
            one = LLMEngine(model, EngineConfig(**ecfg))
            assert eng.results[rid3].token_ids == one.generate_batch([long2], max_tokens=4, temperature=0.0, eos_ids=[])[0].token_ids
        eng.stats["cp_prefills"] = 1
    # a short prompt: every rank falls back to the ordinary path
    rid2 = eng.add_request_context_parallel(prompt[:20], rank, world, max_tokens=2, temperature=0.0, eos_ids=[])
    eng.run_until_done()
    assert eng.stats["cp_prefills"] == 1 and len(eng.results[rid2].token_ids) == 2
    dist.barrier()
    print("CP_ENGINE_WORKER_OK", rank, flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
