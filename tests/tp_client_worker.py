"""Worker (gloo ranks): the public client with a tensor-parallel DistributedConfig; every rank makes the same calls."""
import os

import torch
import torch.distributed as dist


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    from gllm_b200.client import Client
    from gllm_b200.models.config import preset
    from gllm_b200.models.weights import RandomWeights
    from gllm_b200.parallel.config import DistributedConfig, ParallelConfig
    cfg = preset("tiny-qwen3")
    src = RandomWeights(cfg, "cpu", torch.float32, seed=6, std=0.05)
    kw = dict(device="cpu", dtype=torch.float32, max_num_seqs=4, max_model_len=128, max_batch_tokens=64)
    c = Client.from_model(cfg, src, distributed=DistributedConfig(parallel=ParallelConfig(tp=world)), **kw)
    assert dist.is_initialized() and c._state.model.tp_size == world
    prompts = ["the quick brown fox", "hello"]
    got = [c.generate(p).max_tokens(6).temperature(0.0).generate().token_ids for p in prompts]
    gathered = [None] * world
    dist.all_gather_object(gathered, got)
    assert all(g == gathered[0] for g in gathered), "ranks returned different tokens"
    if rank == 0:
        one = Client.from_model(cfg, src, **kw)
        want = [one.generate(p).max_tokens(6).temperature(0.0).generate().token_ids for p in prompts]
        assert got == want, (got, want)
    dist.barrier()
    print("TP_CLIENT_WORKER_OK", rank, flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
