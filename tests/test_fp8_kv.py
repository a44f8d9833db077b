"""fp8 (e4m3) KV cache: half the bytes per token; logits stay close to the bf16 / fp32 cache."""
import pytest
import torch

from gllm_b200.engine.batch import ForwardBatch
from gllm_b200.models.config import preset
from gllm_b200.models.decoder import DecoderModel
from gllm_b200.models.weights import RandomWeights


def _run(model, ids, dev, split=24):
    kv = model.alloc_kv_cache(8)

    def fwd(tok, start):
        T = len(tok)
        b = ForwardBatch(token_ids=torch.tensor(tok, dtype=torch.int32, device=dev),
                         positions=torch.arange(start, start + T, dtype=torch.int32, device=dev),
                         slot_mapping=torch.arange(start, start + T, dtype=torch.int32, device=dev),
                         block_tables=torch.arange(8, dtype=torch.int32, device=dev)[None],
                         ctx_lens=torch.tensor([start + T], dtype=torch.int32, device=dev),
                         q_start=torch.tensor([0], dtype=torch.int32, device=dev),
                         q_len=torch.tensor([T], dtype=torch.int32, device=dev), max_q_len=T)
        return model.forward(b, kv)[:, :model.cfg.vocab_size].float().cpu()
    a = fwd(ids[:split], 0)
    b = fwd(ids[split:], split)           # the second chunk attends over the quantised first chunk
    return torch.cat([a, b]), kv


def test_fp8_kv_cache_cpu_oracle():
    cfg = preset("tiny-qwen3")
    src = RandomWeights(cfg, "cpu", torch.float32, seed=6, std=0.05)
    ids = [(11 * i + 5) % cfg.vocab_size for i in range(60)]
    ref, kv_ref = _run(DecoderModel(cfg, src, device="cpu", dtype=torch.float32, max_positions=128), ids, "cpu")
    m8 = DecoderModel(cfg, src, device="cpu", dtype=torch.float32, max_positions=128, kv_dtype=torch.float8_e4m3fn, kv_scale=0.25)
    got, kv8 = _run(m8, ids, "cpu")
    assert kv8[0].dtype == torch.float8_e4m3fn and kv8[0].element_size() * 2 == torch.empty(0, dtype=torch.bfloat16).element_size()
    deq = kv8[0].float() * 0.25
    assert (deq[:3] - kv_ref[0][:3]).abs().max() < 0.07 * kv_ref[0][:3].abs().max()
    cos = torch.nn.functional.cosine_similarity(got.flatten(), ref.flatten(), dim=0).item()
    assert cos > 0.995, cos


@pytest.mark.gpu
def test_fp8_kv_cache_gpu_matches_cpu():
    cfg = preset("tiny-qwen3")
    src = RandomWeights(cfg, "cpu", torch.float32, seed=6, std=0.05)
    ids = [(11 * i + 5) % cfg.vocab_size for i in range(60)]
    kw = dict(max_positions=128, kv_dtype=torch.float8_e4m3fn, kv_scale=0.25)
    cpu, _ = _run(DecoderModel(cfg, src, device="cpu", dtype=torch.float32, **kw), ids, "cpu")
    gpu, kv = _run(DecoderModel(cfg, src, device="cuda", dtype=torch.bfloat16, **kw), ids, "cuda")
    assert kv[0].dtype == torch.float8_e4m3fn
    cos = torch.nn.functional.cosine_similarity(gpu.flatten(), cpu.flatten(), dim=0).item()
    assert cos > 0.99, cos
