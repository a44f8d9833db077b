"""Worker: the serving engine as pipeline stages (torchrun; gloo on CPU, nccl on GPUs). Every rank runs an LLMEngine
over its stage's layers with the same requests; the tokens must equal a single-process engine's."""
import os
import sys

import torch


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
    from gllm_b200.engine.executor import EngineConfig, LLMEngine
    from gllm_b200.engine.pp import build_pipeline
    from gllm_b200.models.config import preset
    from gllm_b200.models.decoder import DecoderModel
    from gllm_b200.models.weights import RandomWeights
    from gllm_b200.parallel.pipeline import PipelineConfig
    cfg = preset("tiny-qwen3")
    cfg.num_layers = 4
    src = RandomWeights(cfg, "cpu", torch.float32, seed=9, std=0.06)
    pp = build_pipeline(comm, pp=comm.world_size)
    layers = PipelineConfig(num_layers=cfg.num_layers, num_stages=pp.num_stages).stage_ranges()[pp.stage]
    model = DecoderModel(cfg, src, device=dev, dtype=dtype, max_positions=256, layers=layers)
    ec = dict(max_num_seqs=4, max_model_len=128, max_batch_tokens=64, prefill_chunk=32, num_pages=48)
    eng = LLMEngine(model, EngineConfig(**ec), pp=pp)
    g = torch.Generator().manual_seed(2)
    prompts = [torch.randint(0, 1000, (n,), generator=g).tolist() for n in (5, 40, 23, 61, 9)]    # 61 > chunk: chunked prefill
    got = [r.token_ids for r in eng.generate_batch(prompts, max_tokens=7, temperature=0.0, eos_ids=[])]
    if comm.rank == 0:
        full = DecoderModel(cfg, src, device=dev, dtype=dtype, max_positions=256)
        want = [r.token_ids for r in LLMEngine(full, EngineConfig(**ec)).generate_batch(prompts, max_tokens=7, temperature=0.0, eos_ids=[])]
        if mode == "cpu":
            assert got == want, (got, want)
        else:
            assert [g_[:2] for g_ in got] == [w[:2] for w in want], (got, want)
    assert pp.is_last or pp.stats["sent_bytes"] > 0
    assert len(eng.kv_caches) == len(layers)          # a stage holds the KV of its own layers only
    comm.barrier()
    print("PP_ENGINE_WORKER_OK", comm.rank, flush=True)
    if mode != "cpu":
        os._exit(0)
    comm.destroy()


if __name__ == "__main__":
    main()
