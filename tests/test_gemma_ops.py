import math

import torch

from gllm_b200.models import gemma_ops as G
from gllm_b200.models.config import preset


def test_norms_and_dual_rope():
    x = torch.randn(5, 4, 64) * 3
    q = G.qk_norm_weightless(x)
    torch.testing.assert_close(q.pow(2).mean(-1), torch.ones(5, 4), rtol=1e-3, atol=1e-3)
    torch.testing.assert_close(G.value_norm(x).pow(2).mean(-1), torch.ones(5, 4), rtol=1e-3, atol=1e-3)
    assert [l for l in range(10) if G.layer_uses_global_rope(l)] == [4, 9]
    assert G.dual_rope_theta(3, 1e6, 1e4) == 1e4 and G.dual_rope_theta(4, 1e6, 1e4) == 1e6
    cfg = preset("tiny-llama")
    cfg.rope_local_theta = 100.0
    cg, sg, cl, sl = G.build_dual_rope_tables(cfg, 32)
    assert cg.shape == cl.shape and not torch.allclose(cg[5], cl[5])


def test_laurel_altup_and_ple():
    torch.manual_seed(0)
    T, H, n = 6, 16, 4
    x, a = torch.randn(T, H), torch.randn(T, H)
    lw = G.LaurelWeights(torch.zeros(4, H), torch.zeros(H, 4), torch.ones(H))
    torch.testing.assert_close(G.laurel(x, a, lw), (x + a) / math.sqrt(2))          # zero low-rank branch
    lw = G.LaurelWeights(torch.randn(4, H), torch.randn(H, 4), torch.ones(H))
    assert not torch.allclose(G.laurel(x, a, lw), (x + a) / math.sqrt(2))
    w = G.AltUpWeights(router=torch.randn(n, H), predict=torch.zeros(n * n, n), correct=torch.zeros(n, n),
                       router_norm=torch.ones(H), out_scale=torch.ones(H))
    streams = torch.randn(n, T, H)
    pred = G.altup_predict(streams, w)
    torch.testing.assert_close(pred, streams)                                         # zero predictor = identity
    act = streams[0] + 1.0
    cor = G.altup_correct(pred, act, w)
    torch.testing.assert_close(cor[0], act)                                           # active stream takes the layer output
    torch.testing.assert_close(cor[2], streams[2] + 1.0)                              # innovation spread with coefficient 1
    w.predict = torch.randn(n * n, n) * 0.1
    assert not torch.allclose(G.altup_predict(streams, w), streams)
    table = torch.arange(10 * 3 * 4, dtype=torch.float32).reshape(10, 12)
    e = G.ple_gather(table, torch.tensor([2, 7]), layer=1, num_layers=3)
    torch.testing.assert_close(e, table[[2, 7], 4:8] * 2.0)
    inj = G.altup_inject(cor, e.new_ones(T, H), w)
    torch.testing.assert_close(inj[0], cor[0]); torch.testing.assert_close(inj[1], cor[1] + 1.0)


def test_logit_softcap_in_the_gemm_op_cpu():
    """ops.gemm(softcap=c) == c * tanh(x / c) on the CPU oracle path (the CUDA path does it in the GEMM epilogue)."""
    import torch
    from gllm_b200 import ops
    torch.manual_seed(0)
    a = torch.randn(5, 64).to(torch.bfloat16)
    w = torch.randn(32, 64).to(torch.bfloat16)
    got = ops.gemm(a, w, out_dtype=torch.float32, softcap=7.0)
    x = a.float() @ w.float().t()
    torch.testing.assert_close(got, torch.tanh(x / 7.0) * 7.0)
