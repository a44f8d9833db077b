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
    dist.barrier()
    print("TP_MOE_WORKER_OK", rank, flush=True)
    if mode != "cpu":
        os._exit(0)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
