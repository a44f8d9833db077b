"""MoE kernels and the fused MoE decoder path on a B200 against the CPU oracle (run with -m gpu)."""
import pytest
import torch

from gllm_b200.models.config import preset
from gllm_b200.models.decoder import DecoderModel
from gllm_b200.models.weights import RandomWeights
from gllm_b200.ops import moe as M

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.mark.parametrize("E,k,scoring", [(128, 8, "softmax"), (8, 2, "softmax"), (256, 8, "sigmoid"), (60, 4, "softmax")])
def test_route_kernel(E, k, scoring):
    torch.manual_seed(0)
    lg = torch.randn(300, E, device=DEV) * 2
    bias = torch.randn(E, device=DEV) * 0.1 if scoring == "sigmoid" else None
    ids, w = M.route(lg, k, scoring=scoring, sel_bias=bias, scale=1.5)
    rid, rw = M.route_ref(lg.cpu(), k, True, scoring, None if bias is None else bias.cpu(), 1.5)
    assert torch.equal(ids.cpu(), rid)
    torch.testing.assert_close(w.cpu(), rw, rtol=1e-4, atol=1e-6)


def test_permute_combine_kernels():
    torch.manual_seed(1)
    T, k, H, E = 300, 8, 256, 32
    x = torch.randn(T, H, device=DEV).to(torch.bfloat16)
    ss = x.float().pow(2).sum(-1, keepdim=True).contiguous()
    ids = torch.randint(0, E, (T, k), dtype=torch.int32, device=DEV)
    ws = M.MoeWorkspace(T, k, H, 64, E, torch.device(DEV), torch.bfloat16)
    for _ in range(2):  # buffers are reused between calls
        M.permute(x, ss, ids, ws, 0, E)
    offs = ws.offsets.cpu().tolist()
    counts = torch.bincount(ids.reshape(-1).cpu().long(), minlength=E)
    assert offs == [0] + torch.cumsum((counts + 127) // 128 * 128, 0).tolist()
    dest = ws.dest[:T * k].reshape(T, k).cpu()
    assert len(set(dest.reshape(-1).tolist())) == T * k
    a = ws.a_perm.cpu()
    blk = ws.blk_group.cpu()
    for t in range(0, T, 17):
        for j in range(k):
            d, e = int(dest[t, j]), int(ids[t, j])
            assert offs[e] <= d < offs[e + 1] and torch.equal(a[d], x[t].cpu()) and int(blk[d // 128]) == e
            assert abs(float(ws.ss_perm[d, 0]) - float(ss[t, 0])) < 1e-3 * float(ss[t, 0])
    y = torch.randn(ws.max_rows, H, device=DEV).to(torch.bfloat16)
    w = torch.rand(T, k, device=DEV)
    sh = torch.randn(T, H, device=DEV).to(torch.bfloat16)
    xo = x.clone()
    sso = torch.zeros(T, 1, device=DEV)
    M.combine(xo, y, ws.dest, w, shared=sh, ss_out=sso)
    ref = x.float() + sh.float() + (y[dest.to(DEV).long()].float() * w[..., None]).sum(1)
    torch.testing.assert_close(xo.float(), ref, rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(sso[:, 0], xo.float().pow(2).sum(-1), rtol=1e-3, atol=1e-3)


def test_moe_decoder_fused_matches_cpu_oracle():
    from gllm_b200.engine.batch import ForwardBatch
    cfg = preset("tiny-moe")
    cfg.num_shared_experts = 1
    src = RandomWeights(cfg, "cpu", torch.float32, seed=2, std=0.05)
    ref = DecoderModel(cfg, src, device="cpu", dtype=torch.float32, max_positions=256)
    gpu = DecoderModel(cfg, src, device=DEV, dtype=torch.bfloat16, max_positions=256)
    assert gpu.fused
    T = 70
    ids = torch.randint(0, cfg.vocab_size, (T,), dtype=torch.int32)

    def run(m, dev):
        kv = m.alloc_kv_cache(8)
        b = ForwardBatch(token_ids=ids.to(dev), positions=torch.arange(T, dtype=torch.int32, device=dev),
                         slot_mapping=torch.arange(T, dtype=torch.int32, device=dev),
                         block_tables=torch.arange(8, dtype=torch.int32, device=dev)[None],
                         ctx_lens=torch.tensor([T], dtype=torch.int32, device=dev),
                         q_start=torch.tensor([0], dtype=torch.int32, device=dev),
                         q_len=torch.tensor([T], dtype=torch.int32, device=dev), max_q_len=T)
        return m.forward(b, kv)[:, :cfg.vocab_size].float().cpu()
    a, b = run(gpu, torch.device(DEV)), run(ref, torch.device("cpu"))
    cos = torch.nn.functional.cosine_similarity(a.flatten(), b.flatten(), dim=0).item()
    assert cos > 0.995, cos
    assert (a.argmax(-1) == b.argmax(-1)).float().mean() > 0.8


@pytest.mark.parametrize("name", ["tiny-qwen3", "tiny-llama"])
def test_dense_decoder_fused_matches_cpu_oracle(name):
    """Whole fused GPU forward (bf16) against the fp32 CPU oracle, layer by layer."""
    from gllm_b200.engine.batch import ForwardBatch
    cfg = preset(name)
    src = RandomWeights(cfg, "cpu", torch.float32, seed=3, std=0.05)
    ref = DecoderModel(cfg, src, device="cpu", dtype=torch.float32, max_positions=256)
    gpu = DecoderModel(cfg, src, device=DEV, dtype=torch.bfloat16, max_positions=256)
    assert gpu.fused
    T = 150
    ids = torch.randint(0, cfg.vocab_size, (T,), dtype=torch.int32)

    def run(m, dev):
        kv = m.alloc_kv_cache(12)
        b = ForwardBatch(token_ids=ids.to(dev), positions=torch.arange(T, dtype=torch.int32, device=dev),
                         slot_mapping=torch.arange(T, dtype=torch.int32, device=dev),
                         block_tables=torch.arange(12, dtype=torch.int32, device=dev)[None],
                         ctx_lens=torch.tensor([T], dtype=torch.int32, device=dev),
                         q_start=torch.tensor([0], dtype=torch.int32, device=dev),
                         q_len=torch.tensor([T], dtype=torch.int32, device=dev), max_q_len=T)
        lg = m.forward(b, kv, capture_layers=set(range(cfg.num_layers)))
        return lg[:, :cfg.vocab_size].float().cpu(), {k: v.float().cpu() for k, v in m.captured.items()}
    la, ca = run(gpu, torch.device(DEV))
    lb, cb = run(ref, torch.device("cpu"))
    for l in ca:
        assert not torch.isnan(ca[l]).any()
        cos = torch.nn.functional.cosine_similarity(ca[l].flatten(), cb[l].flatten(), dim=0).item()
        assert cos > 0.998, (l, cos)
    assert torch.nn.functional.cosine_similarity(la.flatten(), lb.flatten(), dim=0).item() > 0.995
    assert (la.argmax(-1) == lb.argmax(-1)).float().mean() > 0.85
