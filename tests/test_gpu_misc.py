"""Bandwidth-bound kernels and the sampler vs fp32 references (run with -m gpu on a B200)."""
import pytest
import torch

from gllm_b200 import ops
from gllm_b200.ops import linear as L

pytestmark = pytest.mark.gpu
DEV = "cuda"


def test_embed_gather():
    torch.manual_seed(0)
    table = torch.randn(1000, 576, device=DEV).to(torch.bfloat16)
    ids = torch.randint(0, 1000, (37,), device=DEV, dtype=torch.int32)
    ss = torch.zeros(37, device=DEV)
    out = ops.embed_gather(ids, table, ss_out=ss)
    assert torch.equal(out, table[ids.long()])
    torch.testing.assert_close(ss, out.float().pow(2).sum(-1), rtol=1e-4, atol=1e-4)


def test_rmsnorm_layernorm_glu():
    torch.manual_seed(1)
    x = torch.randn(33, 1536, device=DEV).to(torch.bfloat16)
    r = torch.randn(33, 1536, device=DEV).to(torch.bfloat16)
    w, b = torch.rand(1536, device=DEV) + 0.5, torch.randn(1536, device=DEV)
    h = torch.empty_like(x)
    y = ops.rmsnorm(x, w, 1e-5, residual=r, h_out=h)
    hr = (x.float() + r.float()).to(torch.bfloat16)
    assert torch.equal(h, hr)
    yr = hr.float() * torch.rsqrt(hr.float().pow(2).mean(-1, keepdim=True) + 1e-5) * w
    torch.testing.assert_close(y.float(), yr, rtol=2e-2, atol=2e-2)
    y2 = ops.layernorm(x, w, b, 1e-5)
    torch.testing.assert_close(y2.float(), torch.nn.functional.layer_norm(x.float(), (1536,), w, b, 1e-5),
                               rtol=2e-2, atol=2e-2)
    gu = torch.randn(20, 2 * 768, device=DEV).to(torch.bfloat16)
    g = ops.glu(gu, 0)
    torch.testing.assert_close(g.float(), torch.nn.functional.silu(gu[:, :768].float()) * gu[:, 768:].float(),
                               rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("D,rot", [(64, 64), (128, 128), (96, 48), (256, 256)])
def test_rope_kv_write(D, rot):
    torch.manual_seed(2)
    M, n_q, n_kv, pages, max_pos = 45, 6, 2, 8, 256
    qkv = torch.randn(M, (n_q + 2 * n_kv) * D, device=DEV).to(torch.bfloat16)
    inv = 1.0 / (10000.0 ** (torch.arange(0, rot, 2, device=DEV).double() / rot))
    ang = torch.arange(max_pos, device=DEV).double()[:, None] * inv[None]
    cos_t, sin_t = ang.cos().float().contiguous(), ang.sin().float().contiguous()
    pos = torch.randint(0, max_pos, (M,), device=DEV, dtype=torch.int32)
    slots = torch.randperm(pages * 16, device=DEV)[:M].to(torch.int32)
    qn, kn = torch.rand(D, device=DEV) + 0.5, torch.rand(D, device=DEV) + 0.5
    kv = torch.zeros(pages, 2, n_kv, 16, D, device=DEV, dtype=torch.bfloat16)
    q_out = torch.zeros(M, n_q * D, device=DEV, dtype=torch.bfloat16)
    ops.rope_kv_write(qkv, n_q=n_q, n_kv=n_kv, head_dim=D, rot_dim=rot, positions=pos, slot_mapping=slots,
                      cos_t=cos_t, sin_t=sin_t, q_out=q_out, kv_cache=kv, q_norm_w=qn, k_norm_w=kn)
    q, k, v = L.qkv_post_ref(qkv, n_q, n_kv, D, pos, cos_t, sin_t, qn, kn, 1e-6)
    torch.testing.assert_close(q_out.float(), q.reshape(M, -1), rtol=3e-2, atol=3e-2)
    kv_ref = torch.zeros_like(kv)
    L.kv_write_ref(kv_ref, k, v, slots)
    torch.testing.assert_close(kv.float(), kv_ref.float(), rtol=3e-2, atol=3e-2)


def test_argmax_and_greedy():
    torch.manual_seed(3)
    lg = torch.randn(16, 151936, device=DEV)
    lg[2, 5] = float("nan")
    lg[3, 100] = lg[3, 7] = 50.0
    out = ops.argmax(lg)
    ref = torch.where(torch.isnan(lg), torch.full_like(lg, float("-inf")), lg).argmax(-1)
    assert torch.equal(out.long(), ref)
    assert int(out[3]) == 7
    params = torch.zeros(16, 4, device=DEV)
    assert torch.equal(ops.sample(lg, params).long(), ref)
    assert torch.equal(ops.argmax(lg.to(torch.bfloat16), vocab=1000).long(),
                       lg.to(torch.bfloat16)[:, :1000].float().nan_to_num(float("-inf")).argmax(-1))


def test_sampler_distribution():
    """Empirical token frequencies follow the top-k / top-p filtered softmax of the reference order."""
    torch.manual_seed(4)
    V, B = 512, 4096
    row = torch.randn(V, device=DEV) * 2
    lg = row[None].expand(B, V).contiguous()
    for (t, k, p) in [(0.7, 0, 1.0), (1.0, 20, 1.0), (0.9, 0, 0.8), (1.3, 50, 0.6)]:
        params = torch.tensor([t, k, p, 0], device=DEV).repeat(B, 1).contiguous()
        offs = torch.arange(B, device=DEV, dtype=torch.int64)
        toks = ops.sample(lg, params, seed=1234, step_offsets=offs)
        freq = torch.bincount(toks.long(), minlength=V).float() / B
        want = ops.filtered_probs_ref(row.cpu(), t, k, p).to(DEV)
        assert float(freq[want == 0].sum()) < 2e-3, "sampled a filtered-out token"
        assert float((freq - want).abs().sum()) < 0.2, f"total variation too large for {(t, k, p)}"


def test_pool():
    h = torch.randn(30, 64, device=DEV).to(torch.bfloat16)
    st = torch.tensor([0, 10], dtype=torch.int32, device=DEV)
    ln = torch.tensor([10, 20], dtype=torch.int32, device=DEV)
    out = ops.pool(h, st, ln, "mean")
    torch.testing.assert_close(out[1], h[10:30].float().mean(0), rtol=1e-3, atol=1e-3)
    assert torch.equal(ops.pool(h, st, ln, "cls")[1], h[10].float())
    assert torch.equal(ops.pool(h, st, ln, "last")[0], h[9].float())


@pytest.mark.parametrize("fused", [True, False])
def test_shared_kv_donor_layers_on_the_gpu(fused):
    """A model whose last two layers reuse layer 1's KV pages (query-only QKV GEMM, n_kv = 0) gives the CPU oracle's
    logits, for a prefill and for a decode step over the aliased caches."""
    from gllm_b200.engine.batch import ForwardBatch
    from gllm_b200.models.config import ModelConfig
    from gllm_b200.models.decoder import DecoderModel
    from gllm_b200.models.weights import RandomWeights
    cfg = ModelConfig(arch="llama", hidden_size=256, num_layers=4, num_heads=2, num_kv_heads=1, head_dim=128,
                      intermediate_size=512, vocab_size=300, max_position_embeddings=128, rms_norm_eps=1e-6,
                      num_kv_shared_layers=2)
    models = {}
    for dev in ("cpu", "cuda"):
        src = RandomWeights(cfg, "cpu", torch.bfloat16, seed=0, std=0.05)
        models[dev] = DecoderModel(cfg, src, device=dev, dtype=torch.bfloat16, fused=fused, max_positions=128)
    ids = [5, 17, 250, 3, 99, 42, 7, 11, 200]

    def run(m, toks, kv, start, decode):
        dev = m.device
        n, total = len(toks), start + len(toks)
        i32 = dict(dtype=torch.int32, device=dev)
        fb = ForwardBatch(token_ids=torch.tensor(toks, **i32), positions=torch.arange(start, total, **i32),
                          slot_mapping=torch.arange(start, total, **i32), block_tables=torch.arange(8, **i32)[None],
                          ctx_lens=torch.tensor([total], **i32), is_decode=decode, q_start=torch.tensor([0], **i32),
                          q_len=torch.tensor([n], **i32), max_q_len=n,
                          logits_rows=torch.tensor([n - 1], dtype=torch.int64, device=dev))
        return m.forward(fb, kv).float()[0, :300].cpu()

    out = {}
    for dev, m in models.items():
        kv = m.alloc_kv_cache(8)
        assert kv[2] is kv[1]
        pre = run(m, ids[:-1], kv, 0, False)
        dec = run(m, ids[-1:], kv, len(ids) - 1, True)
        out[dev] = (pre, dec)
    for a, b in zip(out["cuda"], out["cpu"]):
        assert torch.nn.functional.cosine_similarity(a, b, dim=0) > 0.995


@pytest.mark.gpu
@pytest.mark.parametrize("rank", [0, 1, 2])
def test_context_parallel_shard_on_one_gpu(rank):
    """One rank's part of a three-rank context-parallel prefill on a single GPU: the other ranks' KV pages are put
    into the cache by the test (from a whole-prompt prefill) where the all-gather would deliver them; the shard's
    last-row logits and K/V pages must equal the whole-prompt run (tcgen05 prefill attention with a context longer
    than the query, and sequences without any token on this rank)."""
    from gllm_b200.engine.batch import ForwardBatch
    from gllm_b200.models.config import preset
    from gllm_b200.models.decoder import DecoderModel
    from gllm_b200.models.weights import RandomWeights
    from gllm_b200.ops import _native as nv
    from gllm_b200.parallel.context_parallel import CpConfig, CpPrefill
    dev = torch.device("cuda")
    cfg = preset("tiny-qwen3")
    cfg.hidden_size, cfg.num_heads, cfg.num_kv_heads, cfg.head_dim = 512, 4, 2, 128
    cfg.intermediate_size, cfg.num_layers, cfg.vocab_size = 768, 3, 1024
    src = RandomWeights(cfg, "cpu", torch.float32, seed=5, std=0.05)
    model = DecoderModel(cfg, src, device=dev, dtype=torch.bfloat16, max_positions=512)
    lens, pages = [300, 40, 129], 64
    perm = torch.randperm(pages, generator=torch.Generator().manual_seed(3))
    bt = torch.stack([perm[i * 20:(i + 1) * 20] for i in range(len(lens))]).to(torch.int32).to(dev)
    prompts = [((torch.arange(L) * (7 + i) + 3) % cfg.vocab_size).tolist() for i, L in enumerate(lens)]
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
    toks, pos, slots, qs, n = [], [], [], [], 0
    btc = bt.cpu()
    for s_, L in enumerate(lens):
        qs.append(n)
        for t in range(L):
            toks.append(prompts[s_][t]); pos.append(t); slots.append(int(btc[s_, t // 16]) * 16 + t % 16)
        n += L
    kv_ref = model.alloc_kv_cache(pages)
    full = ForwardBatch(token_ids=i32(toks), positions=i32(pos), slot_mapping=i32(slots), block_tables=bt, ctx_lens=i32(lens),
                        q_start=i32(qs), q_len=i32(lens), max_q_len=max(lens))
    want_all = model.forward(full, kv_ref)[:, :cfg.vocab_size].float()

    class OneRank(CpPrefill):
        def exchange(self, kv):      # what the all-gather delivers: the pages the other ranks wrote
            ref = by_ptr[kv.data_ptr()]
            for r in range(self.cfg.cp_size):
                if r != self.cfg.cp_rank and len(self.rank_pages[r]):
                    kv.index_copy_(0, self._idx[r], ref.index_select(0, self._idx[r]))

    cp = OneRank(CpConfig(3, rank), lens, bt)
    kv_cp = model.alloc_kv_cache(pages)
    by_ptr = {a.data_ptr(): b for a, b in zip(kv_cp, kv_ref)}
    batch = cp.local_batch(prompts)
    got = model.forward(batch, kv_cp)[:, :cfg.vocab_size].float()
    torch.cuda.synchronize()
    for s_, L in enumerate(lens):
        t0, t1 = cp.bounds[s_][rank]
        if t1 > t0:      # this rank's last row of the sequence is token t1 - 1
            torch.testing.assert_close(got[s_], want_all[qs[s_] + t1 - 1], rtol=0.05, atol=0.05)
    used = torch.cat([btc[s_, :(L + 15) // 16] for s_, L in enumerate(lens)]).long().to(dev)
    for a, b in zip(kv_cp, kv_ref):
        torch.testing.assert_close(a.float().index_select(0, used), b.float().index_select(0, used), rtol=0.05, atol=0.05)
    assert nv.device_error() == 0
