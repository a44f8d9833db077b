"""Worker: context-parallel prefill (page-aligned shards, KV pages exchanged after every layer's K/V write) against
the same prompts prefilled by one rank. Argument: ``cpu`` (gloo ranks, fp32) or ``cuda`` (NCCL ranks, bf16)."""
import os
import sys

import torch
import torch.distributed as dist


def main():
    mode = sys.argv[1] if len(sys.argv) > 1 else "cpu"
    zigzag = mode.endswith("_zigzag")
    mode = mode.replace("_zigzag", "")
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    cpu = mode == "cpu"
    if cpu:
        dev = torch.device("cpu")
        dist.init_process_group("gloo")
    else:
        torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
        dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
        dist.init_process_group("nccl", device_id=dev)
    from gllm_b200.engine.batch import ForwardBatch
    from gllm_b200.models.config import preset
    from gllm_b200.models.decoder import DecoderModel
    from gllm_b200.models.weights import RandomWeights
    from gllm_b200.parallel.context_parallel import CpConfig, CpPrefill
    cfg = preset("tiny-qwen3")
    cfg.hidden_size, cfg.num_heads, cfg.num_kv_heads, cfg.head_dim = 512, 4, 2, 128
    cfg.intermediate_size, cfg.num_layers, cfg.vocab_size = 768, 3, 1024
    dt = torch.float32 if cpu else torch.bfloat16
    src = RandomWeights(cfg, "cpu", torch.float32, seed=5, std=0.05)
    model = DecoderModel(cfg, src, device=dev, dtype=dt, max_positions=512)
    lens = [300, 70, 129]
    pages = 64
    g = torch.Generator().manual_seed(3)
    perm = torch.randperm(pages, generator=g)
    bt = torch.stack([perm[i * 20:(i + 1) * 20] for i in range(len(lens))]).to(torch.int32).to(dev)
    prompts = [((torch.arange(L) * (7 + i) + 3) % cfg.vocab_size).tolist() for i, L in enumerate(lens)]

    # context parallel: this rank's shard of every prompt
    cp = CpPrefill(CpConfig(world, rank), lens, bt, zigzag=zigzag)
    if zigzag and world == 2:      # rank 0 takes the first and the last quarter of the long prompt
        assert [len(c) for c in cp.chunks[0]] == [2, 2] and cp.owner[0] == 0
    kv_cp = model.alloc_kv_cache(pages)
    local = model.forward(cp.local_batch(prompts), kv_cp)[:, :cfg.vocab_size].float()
    got = cp.last_logits(local)

    # one rank prefills everything
    def i32(v):
        return torch.tensor(v, dtype=torch.int32, device=dev)
    toks, pos, slots, qs, n = [], [], [], [], 0
    btc = bt.cpu()
    for s, L in enumerate(lens):
        qs.append(n)
        for t in range(L):
            toks.append(prompts[s][t]); pos.append(t); slots.append(int(btc[s, t // 16]) * 16 + t % 16)
        n += L
    rows = torch.tensor([qs[s] + lens[s] - 1 for s in range(len(lens))], dtype=torch.long, device=dev)
    full = ForwardBatch(token_ids=i32(toks), positions=i32(pos), slot_mapping=i32(slots), block_tables=bt, ctx_lens=i32(lens),
                        q_start=i32(qs), q_len=i32(lens), max_q_len=max(lens), logits_rows=rows)
    kv_ref = model.alloc_kv_cache(pages)
    want = model.forward(full, kv_ref)[:, :cfg.vocab_size].float()
    tol = dict(rtol=1e-3, atol=2e-4) if cpu else dict(rtol=0.05, atol=0.05)
    torch.testing.assert_close(got.cpu(), want.cpu(), **tol)
    # every rank holds the whole prompts' K/V
    used = torch.cat([btc[s, :(L + 15) // 16] for s, L in enumerate(lens)]).long().to(dev)
    for a, b in zip(kv_cp, kv_ref):
        torch.testing.assert_close(a.float().index_select(0, used).cpu(), b.float().index_select(0, used).cpu(), **tol)
    assert cp.local_batch(prompts).num_tokens < sum(lens)
    if not cpu:
        from gllm_b200.ops import _native as nv
        torch.cuda.synchronize()
        assert nv.device_error() == 0
    dist.barrier()
    print("CP_WORKER_OK", rank, mode, flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
