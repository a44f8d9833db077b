"""Worker (2 gloo ranks): rank 0 verifies with the target model inside the serving engine, rank 1 drafts with another
model; the tokens equal plain greedy decoding of the target. Argument: ``same`` (draft = target weights: every draft
is accepted) or ``other`` (a different draft model: drafts are partly rejected)."""
import os
import sys

import torch
import torch.distributed as dist


def main():
    how = sys.argv[1] if len(sys.argv) > 1 else "same"
    rank = int(os.environ["RANK"])
    dist.init_process_group("gloo")
    from gllm_b200.engine.executor import EngineConfig, LLMEngine
    from gllm_b200.models.config import preset
    from gllm_b200.models.decoder import DecoderModel
    from gllm_b200.models.weights import RandomWeights
    from gllm_b200.parallel.comm import CommHandle
    from gllm_b200.parallel.pd import SaguaroLink
    from gllm_b200.speculative.saguaro import attach_remote_drafts, run_draft_rank
    cfg = preset("tiny-qwen3")
    link = SaguaroLink(CommHandle.from_env("gloo"), draft_rank=1, verify_rank=0, max_draft=8)
    prompt = ((torch.arange(21) * 17 + 3) % cfg.vocab_size).tolist()
    if rank == 1:
        seed = 4 if how == "same" else 9
        draft_model = DecoderModel(cfg, RandomWeights(cfg, "cpu", torch.float32, seed=seed, std=0.05), device="cpu",
                                   dtype=torch.float32, max_positions=128)
        st = run_draft_rank(draft_model, link, k=4)
        assert st["rounds"] > 0 and st["drafted"] > 0
    else:
        target = DecoderModel(cfg, RandomWeights(cfg, "cpu", torch.float32, seed=4, std=0.05), device="cpu",
                              dtype=torch.float32, max_positions=128)
        ecfg = dict(max_num_seqs=2, max_model_len=96, max_batch_tokens=64, prefill_chunk=64, num_pages=24)
        want = LLMEngine(target, EngineConfig(**ecfg)).generate_batch([prompt], max_tokens=14, temperature=0.0, eos_ids=[])[0].token_ids
        eng = LLMEngine(target, EngineConfig(speculative_tokens=4, **ecfg))
        rid = eng.add_request(prompt, max_tokens=14, temperature=0.0, eos_ids=[])
        src = attach_remote_drafts(eng, rid, link, prompt)
        eng.run_until_done()
        src.close()
        got = eng.results[rid].token_ids
        assert got == want, (got, want)
        st = eng.spec_stats
        assert st["drafted"] > 0 and src.rounds > 0
        if how == "same":
            assert st["accepted"] == st["drafted"] and eng.stats["decode_steps"] < 14      # every draft kept: fewer steps
        else:
            assert st["accepted"] < st["drafted"]
    dist.barrier()
    print("SAGUARO_WORKER_OK", rank, how, flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
