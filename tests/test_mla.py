"""Multi-head latent attention: absorbed form on the latent paged cache vs the un-absorbed per-head reference,
chunked prefill + decode consistency, and (on a GPU) the CUDA kernels vs the fp32 CPU path."""
import pytest
import torch

from gllm_b200.engine.batch import ForwardBatch
from gllm_b200.models.config import preset
from gllm_b200.models.decoder import DecoderModel
from gllm_b200.models.mla import mla_attention_naive
from gllm_b200.models.weights import RandomWeights
from gllm_b200.ops import mla as MLA


def _batch(ids, start, n, pages, dev):
    T = ids.shape[0]
    return ForwardBatch(token_ids=ids.to(dev), positions=torch.arange(start, start + T, dtype=torch.int32, device=dev),
                        slot_mapping=torch.arange(start, start + T, dtype=torch.int32, device=dev),
                        block_tables=torch.arange(pages, dtype=torch.int32, device=dev)[None],
                        ctx_lens=torch.tensor([start + T], dtype=torch.int32, device=dev),
                        q_start=torch.tensor([0], dtype=torch.int32, device=dev),
                        q_len=torch.tensor([T], dtype=torch.int32, device=dev), max_q_len=T)


def test_absorbed_attention_equals_per_head_reference():
    cfg = preset("tiny-mla")
    src = RandomWeights(cfg, "cpu", torch.float32, seed=4, std=0.08)
    m = DecoderModel(cfg, src, device="cpu", dtype=torch.float32, max_positions=128)
    assert m.kv_cache_shape(4) == (4, 16, cfg.kv_lora_rank + cfg.qk_rope_head_dim)
    T = 37
    h = torch.randn(T, cfg.hidden_size)
    kv = m.alloc_kv_cache(4)
    b = _batch(torch.zeros(T, dtype=torch.int32), 0, T, 4, "cpu")
    from gllm_b200.models.mla import mla_attention
    out = torch.zeros(T, m.attn_width)
    got = mla_attention(m, m.layers[0].mla, h, b, kv[0], out)
    want = mla_attention_naive(cfg, src, 0, h, b.positions, m.cos, m.sin, m.scale)
    torch.testing.assert_close(got, want, rtol=1e-4, atol=1e-5)


def test_mla_model_chunked_prefill_and_decode_agree_with_one_shot():
    cfg = preset("tiny-mla")
    src = RandomWeights(cfg, "cpu", torch.float32, seed=6, std=0.06)
    m = DecoderModel(cfg, src, device="cpu", dtype=torch.float32, max_positions=128)
    ids = torch.randint(0, cfg.vocab_size, (41,), dtype=torch.int32)
    kv1 = m.alloc_kv_cache(4)
    full = m.forward(_batch(ids, 0, 41, 4, "cpu"), kv1)[:, :cfg.vocab_size].clone()
    kv2 = m.alloc_kv_cache(4)
    a = m.forward(_batch(ids[:24], 0, 24, 4, "cpu"), kv2)[:, :cfg.vocab_size].clone()
    b = m.forward(_batch(ids[24:40], 24, 16, 4, "cpu"), kv2)[:, :cfg.vocab_size].clone()
    dec = ForwardBatch(token_ids=ids[40:41], positions=torch.tensor([40], dtype=torch.int32),
                       slot_mapping=torch.tensor([40], dtype=torch.int32),
                       block_tables=torch.arange(4, dtype=torch.int32)[None],
                       ctx_lens=torch.tensor([41], dtype=torch.int32), is_decode=True)
    c = m.forward(dec, kv2)[:, :cfg.vocab_size]
    torch.testing.assert_close(torch.cat([a, b, c]), full, rtol=2e-4, atol=2e-4)


@pytest.mark.gpu
def test_mla_kernels_match_cpu():
    dev = torch.device("cuda")
    torch.manual_seed(0)
    d_c, d_r, nh, pages = 512, 64, 16, 24
    seqs = [(5, 70), (1, 33), (40, 40), (1, 1)]          # (q_len, ctx_len)
    T = sum(q for q, _ in seqs)
    q = (torch.randn(T, nh * (d_c + d_r)) * 0.3).to(torch.bfloat16)
    cache = (torch.randn(pages, 16, d_c + d_r) * 0.5).to(torch.bfloat16)
    bt = torch.stack([torch.randperm(pages)[:6] for _ in seqs]).to(torch.int32)
    q_len = torch.tensor([s[0] for s in seqs], dtype=torch.int32)
    ctx = torch.tensor([s[1] for s in seqs], dtype=torch.int32)
    q_start = torch.cat([torch.zeros(1, dtype=torch.int32), q_len.cumsum(0)[:-1].to(torch.int32)])
    row_seq = torch.repeat_interleave(torch.arange(len(seqs), dtype=torch.int32), q_len.long())
    want = MLA.latent_attention_ref(q.float(), cache.float(), bt, q_start, q_len, ctx, nh, d_c, 0.05)
    got = MLA.latent_attention(q.to(dev), cache.to(dev), bt.to(dev), q_start.to(dev), q_len.to(dev), ctx.to(dev),
                               row_seq.to(dev), n_heads=nh, d_v=d_c, scale=0.05)
    torch.testing.assert_close(got.float().cpu(), want, rtol=2e-2, atol=2e-2)
    # latent write
    kv_a = torch.randn(T, d_c + d_r).to(torch.bfloat16)
    nw = 1 + 0.1 * torch.randn(d_c)
    cos, sin = torch.rand(128, d_r // 2), torch.rand(128, d_r // 2)
    pos = torch.randint(0, 128, (T,), dtype=torch.int32)
    slots = torch.randperm(pages * 16)[:T].to(torch.int32)
    slots[3] = -1
    c_cpu = torch.zeros(pages, 16, d_c + d_r)
    MLA.latent_write(kv_a.float(), d_c, nw, 1e-6, pos, slots, cos, sin, c_cpu)
    c_gpu = torch.zeros(pages, 16, d_c + d_r, dtype=torch.bfloat16, device=dev)
    MLA.latent_write(kv_a.to(dev), d_c, nw.to(dev), 1e-6, pos.to(dev), slots.to(dev), cos.to(dev), sin.to(dev), c_gpu)
    torch.testing.assert_close(c_gpu.float().cpu(), c_cpu, rtol=2e-2, atol=2e-2)


@pytest.mark.gpu
def test_mla_model_gpu_matches_cpu_oracle():
    cfg = preset("tiny-mla")
    src = RandomWeights(cfg, "cpu", torch.float32, seed=8, std=0.05)
    ref = DecoderModel(cfg, src, device="cpu", dtype=torch.float32, max_positions=256)
    gpu = DecoderModel(cfg, src, device="cuda", dtype=torch.bfloat16, max_positions=256)
    ids = torch.randint(0, cfg.vocab_size, (90,), dtype=torch.int32)
    a = gpu.forward(_batch(ids, 0, 90, 8, "cuda"), gpu.alloc_kv_cache(8))[:, :cfg.vocab_size].float().cpu()
    b = ref.forward(_batch(ids, 0, 90, 8, "cpu"), ref.alloc_kv_cache(8))[:, :cfg.vocab_size]
    cos = torch.nn.functional.cosine_similarity(a.flatten(), b.flatten(), dim=0).item()
    assert cos > 0.995, cos


def test_mla_moe_model_generates_through_the_client():
    from gllm_b200.client import Client
    cfg = preset("tiny-mla")
    c = Client.from_model(cfg, RandomWeights(cfg, "cpu", torch.float32, seed=3), device="cpu", dtype=torch.float32,
                          max_num_seqs=4, max_model_len=256, max_batch_tokens=48)
    prompt = "the quick brown fox jumps over the lazy dog again and again and again"   # > one prefill chunk
    r1 = c.generate(prompt).max_tokens(5).temperature(0.0).generate()
    r2 = c.generate(prompt).max_tokens(5).temperature(0.0).generate()
    assert r1.token_ids == r2.token_ids and 1 <= len(r1.token_ids) <= 5


@pytest.mark.gpu
@pytest.mark.parametrize("n_heads,splits", [(16, 1), (16, 4), (20, 0), (128, 1), (4, 2)])
def test_mla_tensor_core_decode_matches_reference(n_heads, splits):
    dev = torch.device("cuda")
    torch.manual_seed(3)
    pages = 96
    ctx = torch.tensor([1, 15, 16, 17, 63, 64, 65, 200, 333, 0], dtype=torch.int32)
    B = ctx.numel()
    q = (torch.randn(B, n_heads * 576) * 0.3).to(torch.bfloat16)
    cache = (torch.randn(pages, 16, 576) * 0.5).to(torch.bfloat16)
    bt = torch.stack([torch.randperm(pages)[:24] for _ in range(B)]).to(torch.int32)
    idx = torch.arange(B, dtype=torch.int32)
    want = MLA.latent_attention_ref(q.float(), cache.float(), bt, idx, torch.ones_like(idx), ctx, n_heads, 512, 0.07)
    got = MLA.latent_decode(q.to(dev), cache.to(dev), bt.to(dev), ctx.to(dev), n_heads=n_heads, scale=0.07, splits=splits)
    torch.testing.assert_close(got.float().cpu(), want, rtol=2e-2, atol=2e-2)
    from gllm_b200.ops import _native as nv
    assert nv.device_error() == 0


@pytest.mark.gpu
@pytest.mark.parametrize("causal", [True, False])
def test_mla_tensor_core_prefill_rows_match_reference(causal):
    """Prefill chunks on the tensor-core kernel (one row per query token): whole prompts, a continued chunk whose
    context is longer than its query, a single token; against the fp32 statement of the absorbed attention."""
    dev = torch.device("cuda")
    torch.manual_seed(5)
    nh, pages = 16, 64
    seqs = [(70, 70), (33, 120), (1, 47), (129, 129)]          # (q_len, ctx_len)
    T = sum(s[0] for s in seqs)
    q = (torch.randn(T, nh * 576) * 0.3).to(torch.bfloat16)
    cache = (torch.randn(pages, 16, 576) * 0.5).to(torch.bfloat16)
    bt = torch.stack([torch.randperm(pages)[:10] for _ in seqs]).to(torch.int32)
    q_len = torch.tensor([s[0] for s in seqs], dtype=torch.int32)
    ctx = torch.tensor([s[1] for s in seqs], dtype=torch.int32)
    q_start = torch.cat([torch.zeros(1, dtype=torch.int32), q_len.cumsum(0)[:-1].to(torch.int32)])
    row_seq = torch.repeat_interleave(torch.arange(len(seqs), dtype=torch.int32), q_len.long())
    positions = torch.cat([torch.arange(c - l, c, dtype=torch.int32) for l, c in seqs])
    want = MLA.latent_attention_ref(q.float(), cache.float(), bt, q_start, q_len, ctx, nh, 512, 0.06, causal=causal)
    got = MLA.latent_prefill(q.to(dev), cache.to(dev), bt.to(dev), row_seq.to(dev), positions.to(dev), ctx.to(dev),
                             n_heads=nh, scale=0.06, causal=causal)
    torch.testing.assert_close(got.float().cpu(), want, rtol=2e-2, atol=2e-2)
    from gllm_b200.ops import _native as nv
    assert nv.device_error() == 0
