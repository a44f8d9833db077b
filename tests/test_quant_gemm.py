"""Canonical quantised weights: packers agree with the loaders' dequantisers; the CUDA kernel agrees with
``dequantize()`` (GPU test)."""
import numpy as np
import pytest
import torch

from gllm_b200.loader import pairing, quant
from gllm_b200.loader.quant import BY_NAME
from gllm_b200.ops import quant_gemm as Q


def test_packers_match_loader_dequant():
    torch.manual_seed(0)
    w = torch.randn(64, 256) * 0.1
    q, e = pairing.quantize_mxfp8(w)
    torch.testing.assert_close(Q.from_mxfp8(q, e).dequantize(), pairing.dequant_mxfp8(q, e))
    qb, sinv = pairing.quantize_fp8_block(torch.randn(256, 256) * 0.1)
    torch.testing.assert_close(Q.from_fp8_block(qb, sinv).dequantize(), pairing.dequant_fp8_block(qb, sinv), rtol=8e-3, atol=1e-6)
    qt = (w / 0.01).to(torch.float8_e4m3fn)
    torch.testing.assert_close(Q.from_fp8_tensor(qt, 0.01).dequantize(), pairing.dequant_fp8(qt, torch.tensor(0.01)), rtol=8e-3, atol=1e-6)
    # NVFP4 / MXFP4 test vectors from the block quantisers
    nv_w = torch.randint(0, 256, (16, 64), dtype=torch.uint8)
    nv_s = quant.fp8_e4m3_encode(torch.rand(16, 8) + 0.1)
    got = Q.from_nvfp4(nv_w, nv_s, torch.tensor([0.5])).dequantize()
    torch.testing.assert_close(got, pairing.dequant_nvfp4(nv_w, nv_s, torch.tensor([0.5])), rtol=8e-3, atol=1e-6)
    mx_b = torch.randint(0, 256, (8, 4, 16), dtype=torch.uint8)
    mx_s = torch.randint(120, 130, (8, 4), dtype=torch.uint8)
    torch.testing.assert_close(Q.from_mxfp4(mx_b, mx_s).dequantize(), pairing.dequant_mxfp4_st(mx_b, mx_s))
    # AWQ / GPTQ
    K, N, g = 128, 32, 64
    qw = torch.randint(-2 ** 31, 2 ** 31 - 1, (K, N // 8), dtype=torch.int32)
    sc = (torch.rand(K // g, N) * 0.02 + 0.001).half()
    qz = torch.randint(-2 ** 31, 2 ** 31 - 1, (K // g, N // 8), dtype=torch.int32)
    torch.testing.assert_close(Q.from_awq(qw, sc, qz).dequantize(), pairing.dequant_awq(qw, sc, qz), rtol=1e-2, atol=1e-4)
    gq = torch.randint(-2 ** 31, 2 ** 31 - 1, (K // 8, N), dtype=torch.int32)
    torch.testing.assert_close(Q.from_gptq(gq, sc, qz).dequantize(), pairing.dequant_gptq(gq, sc, qz), rtol=1e-2, atol=1e-4)
    assert Q.from_gptq(gq, sc, qz, g_idx=torch.randperm(K) // g) is None


@pytest.mark.parametrize("tid,enc", [(BY_NAME["Q8_0"].id, quant.quantize_q8_0), (BY_NAME["Q4_0"].id, quant.quantize_q4_0),
                                      (BY_NAME["Q4_K"].id, quant.quantize_q4_k), (BY_NAME["Q6_K"].id, quant.quantize_q6_k)])
def test_gguf_repack_is_exact(tid, enc):
    rng = np.random.default_rng(int(tid))
    n, k = 8, 512
    x = rng.standard_normal((n, k)).astype(np.float32)
    raw = enc(x.reshape(-1))
    want = quant.dequantize(tid, raw, n * k).reshape(n, k).float()
    qw = Q.from_gguf(tid, raw, n, k)
    got = qw.dequantize()
    # the only loss is rounding scale * sub-scale products to bf16
    assert (got - want).abs().max() <= 8e-3 * want.abs().max() + 1e-6
    assert Q.from_gguf(BY_NAME["F16"].id, b"", 1, 1) is None


@pytest.mark.parametrize("mode,group,tol", [("fp8", 32, 0.04), ("int8", 32, 0.01), ("int4", 32, 0.12), ("fp4", 16, 0.2)])
def test_quantisers_and_cpu_qgemm(mode, group, tol):
    torch.manual_seed(1)
    w = torch.randn(96, 128)
    qw = Q.quantize(w, mode, group)
    assert (qw.dequantize() - w).abs().max() < tol * w.abs().max() * 1.6 and qw.nbytes() < w.numel() * 2
    a = torch.randn(5, 128)
    y = Q.qgemm(a, qw)
    torch.testing.assert_close(y, a @ qw.dequantize().t())
    ss = a.pow(2).sum(-1, keepdim=True)
    yn = Q.qgemm(a, qw, row_ss=ss, norm_dim=128, eps=1e-6)
    torch.testing.assert_close(yn, (a * torch.rsqrt(a.pow(2).mean(-1, keepdim=True) + 1e-6)) @ qw.dequantize().t(), rtol=1e-4, atol=1e-4)


@pytest.mark.gpu
@pytest.mark.parametrize("mode,group", [("fp8", 32), ("fp8", 128), ("fp4", 16), ("fp4", 32), ("int4", 32), ("int4", 128), ("int8", 16)])
@pytest.mark.parametrize("M,N,K,splits", [(200, 384, 512, 0), (37, 1024, 2048, 0), (256, 256, 4096, 1), (130, 136, 256, 0)])
def test_qgemm_kernel_matches_dequantised_reference(mode, group, M, N, K, splits):
    dev = torch.device("cuda")
    torch.manual_seed(2)
    w = torch.randn(N, K) * 0.05
    qw = Q.quantize(w, mode, group)
    a = torch.randn(M, K).to(torch.bfloat16)
    want = a.float() @ qw.dequantize().to(torch.bfloat16).float().t()
    got = Q.qgemm(a.to(dev), qw.to(dev), splits=splits).float().cpu()
    err = (got - want).abs().max().item()
    assert err < 0.02 * want.abs().max().item() + 1e-3, (mode, group, err)
    ss = a.float().pow(2).sum(-1, keepdim=True).to(dev)
    gotn = Q.qgemm(a.to(dev), qw.to(dev), row_ss=ss, norm_dim=K, eps=1e-6).float().cpu()
    wantn = want * torch.rsqrt(a.float().pow(2).mean(-1, keepdim=True) + 1e-6)
    assert (gotn - wantn).abs().max().item() < 0.02 * wantn.abs().max().item() + 1e-3
    from gllm_b200.ops import _native as nv
    assert nv.device_error() == 0


def _logits(model, ids, dev):
    from gllm_b200.engine.batch import ForwardBatch
    T = len(ids)
    b = ForwardBatch(token_ids=torch.tensor(ids, dtype=torch.int32, device=dev), positions=torch.arange(T, dtype=torch.int32, device=dev),
                     slot_mapping=torch.arange(T, dtype=torch.int32, device=dev),
                     block_tables=torch.arange(8, dtype=torch.int32, device=dev)[None],
                     ctx_lens=torch.tensor([T], dtype=torch.int32, device=dev), q_start=torch.tensor([0], dtype=torch.int32, device=dev),
                     q_len=torch.tensor([T], dtype=torch.int32, device=dev), max_q_len=T)
    return model.forward(b, model.alloc_kv_cache(8))[:, :model.cfg.vocab_size].float().cpu()


def test_model_with_load_time_quantised_weights_cpu():
    from gllm_b200.models.config import preset
    from gllm_b200.models.decoder import DecoderModel
    from gllm_b200.models.weights import RandomWeights
    cfg = preset("tiny-qwen3")
    src = RandomWeights(cfg, "cpu", torch.float32, seed=4, std=0.05)
    dense = DecoderModel(cfg, src, device="cpu", dtype=torch.float32, max_positions=128)
    ids = list(range(3, 40))
    want = _logits(dense, ids, "cpu")
    for mode, tol in (("int8", 0.999), ("fp8", 0.995), ("int4", 0.96)):
        qm = DecoderModel(cfg, src, device="cpu", dtype=torch.float32, max_positions=128, weight_quant=mode)
        assert isinstance(qm.layers[0].wqkv, Q.QuantWeight) and qm.weight_bytes() < dense.weight_bytes() * (0.4 if mode != "int4" else 0.25)
        got = _logits(qm, ids, "cpu")
        cos = torch.nn.functional.cosine_similarity(got.flatten(), want.flatten(), dim=0).item()
        assert cos > tol, (mode, cos)


@pytest.mark.gpu
@pytest.mark.parametrize("mode", ["fp8", "int4"])
def test_quantised_model_gpu_matches_cpu(mode):
    from gllm_b200.models.config import preset
    from gllm_b200.models.decoder import DecoderModel
    from gllm_b200.models.weights import RandomWeights
    cfg = preset("tiny-qwen3")
    src = RandomWeights(cfg, "cpu", torch.float32, seed=4, std=0.05)
    cpu = DecoderModel(cfg, src, device="cpu", dtype=torch.float32, max_positions=128, weight_quant=mode)
    gpu = DecoderModel(cfg, src, device="cuda", dtype=torch.bfloat16, max_positions=128, weight_quant=mode)
    ids = list(range(3, 80))
    a, b = _logits(gpu, ids, "cuda"), _logits(cpu, ids, "cpu")
    cos = torch.nn.functional.cosine_similarity(a.flatten(), b.flatten(), dim=0).item()
    assert cos > 0.99, cos
