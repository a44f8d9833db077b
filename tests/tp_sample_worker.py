"""Worker (gloo ranks): vocabulary-parallel sampling from per-rank top-k candidates instead of the gathered vocabulary."""
import os

import torch
import torch.distributed as dist


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo")
    from gllm_b200.models.weights import shard_range
    from gllm_b200.parallel.tensor_parallel import TPContext
    tp = TPContext(rank, world, "cpu", mode="nccl", max_tokens=16, hidden=64)
    B, V = 12, 1000 + world      # the shards differ in width
    g = torch.Generator().manual_seed(4)
    full = torch.randn(B, V, generator=g) * 3
    a, b = shard_range(V, rank, world)
    local = full[:, a:b].contiguous()
    params = torch.zeros(B, 4)
    params[:, 0] = 0.8
    params[:, 1] = torch.tensor([1, 1, 2, 5, 8, 8, 20, 40, 50, 64, 3, 0.0])
    params[:, 2] = torch.tensor([1, 1, 1, 1, 0.9, 0.5, 1, 0.95, 1, 0.8, 1, 1.0])
    params[11, 0], params[11, 1] = 0.0, 0.0      # a greedy row inside a sampling batch
    offsets = torch.zeros(B, dtype=torch.int64)
    order = full.argsort(1, descending=True)
    seen = [set() for _ in range(B)]
    for step in range(30):
        out = torch.zeros(B, dtype=torch.int32)
        tp.sample_vocab_parallel(local, b - a, a, params, 7, offsets + step, out, V, greedy=False, topk_cap=64)
        everyone = [torch.zeros_like(out) for _ in range(world)]
        dist.all_gather(everyone, out)
        assert all(torch.equal(everyone[0], e) for e in everyone), "ranks disagree on the sampled tokens"
        for i in range(B):
            k = int(params[i, 1]) or 1
            assert int(out[i]) in order[i, :k].tolist(), f"row {i}: token {int(out[i])} outside the global top-{k}"
            seen[i].add(int(out[i]))
    assert all(len(seen[i]) == 1 and next(iter(seen[i])) == int(order[i, 0]) for i in (0, 1, 11))     # top-1 and greedy rows
    assert len(seen[8]) > 3                                                                           # top-50 at T = 0.8 explores
    dist.barrier()
    print("TP_SAMPLE_WORKER_OK", rank, flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
