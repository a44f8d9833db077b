"""Worker for the pipeline-parallel tests (torchrun; gloo on CPU, nccl on GPUs)."""
import os
import sys

import torch
import torch.distributed as dist


def main():
    mode = sys.argv[1] if len(sys.argv) > 1 else "cpu"
    from gllm_b200.parallel.comm import CommHandle
    if mode == "cpu":
        comm = CommHandle.from_env("gloo", timeout_s=120)
        dev, dtype = torch.device("cpu"), torch.float32
    else:
        local = int(os.environ["LOCAL_RANK"])
        torch.cuda.set_device(local)
        dev, dtype = torch.device("cuda", local), torch.bfloat16
        comm = CommHandle.from_env("nccl", device=dev, timeout_s=120)
    from gllm_b200.engine.batch import ForwardBatch
    from gllm_b200.models.config import preset
    from gllm_b200.models.decoder import DecoderModel
    from gllm_b200.models.weights import RandomWeights
    from gllm_b200.parallel.pipeline.engine import build_stage_runner
    cfg = preset("tiny-qwen3")
    cfg.num_layers = 4
    src = RandomWeights(cfg, "cpu", torch.float32, seed=9, std=0.06)
    pp = comm.world_size
    runner = build_stage_runner(cfg, src, comm, pp=pp, device=dev, dtype=dtype, max_seq_len=64)
    assert len(runner.model.layer_ids) == cfg.num_layers // pp or pp == 3
    prompts = [[5, 6, 7, 8, 9], [100, 101, 102], [7] * 20, [11, 400, 12, 401, 13, 402, 14]]
    got = runner.generate_greedy(prompts, 6, micro_batches=2)
    if comm.rank == 0:
        full = DecoderModel(cfg, src, device=dev, dtype=dtype, max_positions=1024)
        for p, g in zip(prompts, got):
            seq = list(p)
            kv = full.alloc_kv_cache(8)
            for _ in range(6):
                T = len(seq)
                b = ForwardBatch(token_ids=torch.tensor(seq, dtype=torch.int32, device=dev),
                                 positions=torch.arange(T, dtype=torch.int32, device=dev),
                                 slot_mapping=torch.arange(T, dtype=torch.int32, device=dev),
                                 block_tables=torch.arange(8, dtype=torch.int32, device=dev)[None],
                                 ctx_lens=torch.tensor([T], dtype=torch.int32, device=dev),
                                 q_start=torch.tensor([0], dtype=torch.int32, device=dev),
                                 q_len=torch.tensor([T], dtype=torch.int32, device=dev), max_q_len=T)
                seq.append(int(full.forward(b, kv)[-1, :cfg.vocab_size].argmax()))
            want = seq[len(p):]
            if mode == "cpu":
                assert g == want, (g, want)
            else:       # bf16: allow a late divergence, the first tokens must agree
                assert g[:2] == want[:2], (g, want)
        assert runner.stats["sent_bytes"] > 0
    else:
        assert got is None
    comm.barrier()
    print("PP_WORKER_OK", comm.rank, flush=True)
    if mode != "cpu":
        os._exit(0)
    comm.destroy()


if __name__ == "__main__":
    main()
