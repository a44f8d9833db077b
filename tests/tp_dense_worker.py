"""Worker: a tensor-parallel dense decoder on gloo ranks (CPU) compared with the unsplit model. Arguments: number of
heads and of KV heads (fewer KV heads than ranks exercises KV-head replication)."""
import os
import sys

import torch
import torch.distributed as dist


def main():
    n_heads, n_kv = int(sys.argv[1]), int(sys.argv[2])
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo")
    from gllm_b200.engine.batch import ForwardBatch
    from gllm_b200.models.config import preset
    from gllm_b200.models.decoder import DecoderModel
    from gllm_b200.models.weights import RandomWeights
    from gllm_b200.parallel.tensor_parallel import TPContext
    cfg = preset("tiny-qwen3")
    cfg.num_heads, cfg.num_kv_heads, cfg.head_dim, cfg.attention_bias = n_heads, n_kv, 32, True
    src = RandomWeights(cfg, "cpu", torch.float32, seed=3, std=0.05)
    tp = TPContext(rank, world, "cpu", mode="nccl", max_tokens=64, hidden=cfg.hidden_size)
    model = DecoderModel(cfg, src, device="cpu", dtype=torch.float32, tp=tp, max_positions=128)
    assert model.n_kv_local == max(1, n_kv // world)
    T = 37
    ids = (torch.arange(T, dtype=torch.int32) * 5 + 1) % cfg.vocab_size

    def batch():
        return ForwardBatch(token_ids=ids, positions=torch.arange(T, dtype=torch.int32),
                            slot_mapping=torch.arange(T, dtype=torch.int32),
                            block_tables=torch.arange(4, dtype=torch.int32)[None],
                            ctx_lens=torch.tensor([T], dtype=torch.int32), q_start=torch.tensor([0], dtype=torch.int32),
                            q_len=torch.tensor([T], dtype=torch.int32), max_q_len=T)
    local = model.forward(batch(), model.alloc_kv_cache(4))[:, :model.vocab_local].float().contiguous()
    parts = [torch.empty_like(local) for _ in range(world)]
    dist.all_gather(parts, local)
    got = torch.cat(parts, 1)
    if rank == 0:
        ref = DecoderModel(cfg, src, device="cpu", dtype=torch.float32, max_positions=128)
        want = ref.forward(batch(), ref.alloc_kv_cache(4))[:, :cfg.vocab_size]
        torch.testing.assert_close(got, want, rtol=1e-3, atol=1e-4)
    dist.barrier()
    print("TP_DENSE_WORKER_OK", rank, flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
