"""The scalar C++ reference against the PyTorch fp32 model and sampler semantics."""
import torch

from gllm_b200 import ref
from gllm_b200.engine.batch import ForwardBatch
from gllm_b200.models.config import preset
from gllm_b200.models.decoder import DecoderModel
from gllm_b200.models.weights import RandomWeights
from gllm_b200.ops.moe import route_ref


def _torch_logits(model, ids):
    T = len(ids)
    b = ForwardBatch(token_ids=torch.tensor(ids, dtype=torch.int32), positions=torch.arange(T, dtype=torch.int32),
                     slot_mapping=torch.arange(T, dtype=torch.int32), block_tables=torch.arange(8, dtype=torch.int32)[None],
                     ctx_lens=torch.tensor([T], dtype=torch.int32), q_start=torch.tensor([0], dtype=torch.int32),
                     q_len=torch.tensor([T], dtype=torch.int32), max_q_len=T)
    return model.forward(b, model.alloc_kv_cache(8))[:, :model.cfg.vocab_size]


def test_scalar_reference_matches_torch_model():
    for name in ("tiny-llama", "tiny-qwen3"):
        cfg = preset(name)
        src = RandomWeights(cfg, "cpu", torch.float32, seed=5, std=0.05)
        tm = DecoderModel(cfg, src, device="cpu", dtype=torch.float32, max_positions=128)
        cm = ref.CpuReferenceModel(cfg, src, num_pages=8)
        ids = [5, 9, 200, 31, 77, 3, 3, 150, 42, 8, 19, 64, 128, 255, 1, 2, 90, 91]      # crosses a page boundary
        want = _torch_logits(tm, ids)[-1]
        got = cm.forward(ids)
        torch.testing.assert_close(got, want, rtol=2e-4, atol=2e-4)
        cm.reset()
        gen = cm.generate_greedy(ids, 6)
        seq = list(ids)
        for _ in range(6):
            seq.append(int(_torch_logits(tm, seq)[-1].argmax()))
        assert gen == seq[len(ids):]


def test_reference_sampler_and_moe_gate():
    lg = torch.tensor([1.0, 3.0, 2.0, 0.5, 2.9])
    assert ref.sample(lg, 0.0, 0, 1.0, 0.9) == 1
    assert ref.sample(lg, 1.0, 1, 1.0, 0.99) == 1                       # top-k 1
    assert ref.sample(lg, 1.0, 0, 0.3, 0.99) == 1                       # nucleus keeps only the head
    p = torch.softmax(lg[[1, 4]] / 1.0, 0)                               # top-k 2, renormalised
    assert ref.sample(lg, 1.0, 2, 1.0, float(p[0]) - 1e-3) == 1 and ref.sample(lg, 1.0, 2, 1.0, float(p[0]) + 1e-3) == 4
    counts = torch.zeros(5)
    g = torch.Generator().manual_seed(0)
    for _ in range(4000):
        counts[ref.sample(lg, 0.8, 0, 1.0, float(torch.rand((), generator=g)))] += 1
    assert (counts / 4000 - torch.softmax(lg / 0.8, 0)).abs().max() < 0.03
    logits = torch.randn(16)
    ids, w = ref.moe_gate_topk(logits, 4)
    rid, rw = route_ref(logits[None], 4)
    assert ids.tolist() == rid[0].tolist() and torch.allclose(w, rw[0], atol=1e-6)
