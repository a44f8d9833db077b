"""Block-scaled operands (MXFP8 / NVFP4): packers and oracle on CPU; on a B200 (-m gpu) the tcgen05 block-scaled GEMM
with its epilogues and the activation-quantisation kernel against the fp32 product of the SAME quantised operands."""
import pytest
import torch

from gllm_b200.ops import blockscale as bs
from gllm_b200.ops import linear as L


def test_scale_chunk_layout_round_trip_and_byte_positions():
    sf = torch.arange(200 * 10, dtype=torch.int64).remainder(251).to(torch.uint8).view(200, 10)
    buf = bs.sf_swizzle(sf)
    assert buf.numel() == bs.sf_bytes(200, 10) == 2 * 3 * 512
    assert torch.equal(bs.sf_unswizzle(buf, 200, 10), sf)
    for r, c in [(0, 0), (37, 5), (131, 9), (199, 2), (64, 4)]:
        chunk = (r // 128) * 3 + c // 4
        off = chunk * 512 + (r % 32) * 16 + ((r % 128) // 32) * 4 + c % 4
        assert int(buf[off]) == int(sf[r, c])


def test_codecs():
    v = torch.tensor([0.0, 0.5, 0.74, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 7.0, -0.3, -6.0, -2.49])
    dec = bs.e2m1_decode(bs.e2m1_encode(v))
    # ties go to the even code: 0.75 -> 1.0 (code 2), 1.25 -> 1.0, 1.75 -> 2.0, 2.5 -> 2.0, 3.5 -> 4.0, 5.0 -> 4.0
    assert dec.tolist() == [0.0, 0.5, 0.5, 1.0, 1.0, 2.0, 2.0, 4.0, 4.0, 6.0, -0.5, -6.0, -2.0]
    codes = torch.arange(16, dtype=torch.uint8)[None].repeat(2, 1)
    assert torch.equal(bs.unpack_nibbles(bs.pack_nibbles(codes)), codes)
    s = torch.tensor([2.0 ** -20, 1.0, 8.0, 2.0 ** 30])
    assert torch.equal(bs.ue8m0_decode(bs.ue8m0_encode(s)), s)


@pytest.mark.parametrize("fmt", ["mxfp8", "nvfp4"])
def test_quantise_error_bounds_and_oracle_gemm(fmt):
    torch.manual_seed(0)
    x = torch.randn(70, 512) * torch.logspace(-2, 2, 70)[:, None]          # rows of very different magnitude
    q = bs.quantize(x, fmt)
    deq = q.dequantize()[:, :512]
    blk = 32 if fmt == "mxfp8" else 16
    amax = x.view(70, -1, blk).abs().amax(-1).repeat_interleave(blk, 1)
    # e4m3 keeps 3 mantissa bits under a power-of-two scale; e2m1's coarsest step is 2 (between 4 and 6) of 6
    bound = (2.0 ** -3 if fmt == "mxfp8" else 0.26) * amax + 1e-6
    assert ((deq - x).abs() <= bound).all()
    w = torch.randn(96, 512) * 0.05
    wq = bs.quantize(w, fmt)
    got = bs.gemm(q, wq, out_dtype=torch.float32)
    torch.testing.assert_close(got, q.dequantize() @ wq.dequantize().t(), rtol=1e-5, atol=1e-5)
    ref = x @ w.t()
    cos = torch.nn.functional.cosine_similarity(got.flatten(), ref.flatten(), dim=0).item()
    assert cos > (0.998 if fmt == "mxfp8" else 0.97), cos


def test_checkpoint_forms():
    torch.manual_seed(1)
    w = torch.randn(256, 256) * 0.1
    q = bs.quantize_mxfp8(w)
    again = bs.from_mxfp8_checkpoint(q.codes.view(torch.float8_e4m3fn), bs.sf_unswizzle(q.sf, 256, 8))
    assert torch.equal(again.dequantize(), q.dequantize())
    n = bs.quantize_nvfp4(w)
    again = bs.from_nvfp4_checkpoint(n.codes, bs.sf_unswizzle(n.sf, 256, 16), n.tensor_scale)
    assert torch.equal(again.dequantize(), n.dequantize())
    # 128 x 128 block-scaled fp8 with arbitrary fp32 scales is re-quantised to power-of-two block scales
    scale = torch.tensor([[0.013, 0.4], [1.7, 0.09]])
    codes = (w / scale.repeat_interleave(128, 0).repeat_interleave(128, 1)).clamp(-448, 448).to(torch.float8_e4m3fn)
    blk = bs.from_fp8_block_checkpoint(codes, scale)
    want = codes.float() * scale.repeat_interleave(128, 0).repeat_interleave(128, 1)
    assert ((blk.dequantize() - want).abs() <= 2.0 ** -3 * want.abs().view(256, 8, 32).amax(-1).repeat_interleave(32, 1) + 1e-7).all()


# ------------------------------------------------------------------------------------------------
gpu = pytest.mark.gpu


def _rows_close(got, ref, tol=2e-2):
    got, ref = got.float().cpu(), ref.float().cpu()
    err = (got - ref).abs().amax(-1)
    lim = tol * ref.abs().amax(-1).clamp_min(1e-3) + 1e-3
    bad = (err > lim).nonzero().flatten()
    assert bad.numel() == 0, f"rows {bad[:8].tolist()} off by {err[bad[:8]].tolist()} (limit {lim[bad[:8]].tolist()})"


@gpu
@pytest.mark.parametrize("fmt", ["mxfp8", "nvfp4"])
def test_quantize_act_kernel_matches_host_quantiser(fmt):
    dev = torch.device("cuda")
    torch.manual_seed(3)
    x = (torch.randn(300, 1024) * torch.logspace(-1, 1, 300)[:, None]).to(torch.bfloat16)
    ts = 0.01 if fmt == "nvfp4" else 1.0
    q = bs.quantize_act(x.to(dev), fmt, tensor_scale=ts)
    host = bs.quantize_mxfp8(x.float()) if fmt == "mxfp8" else bs.quantize_nvfp4(x.float(), ts)
    rows_sf = 1024 // (32 if fmt == "mxfp8" else 16)
    assert torch.equal(bs.sf_unswizzle(q.sf.cpu(), 300, rows_sf), bs.sf_unswizzle(host.sf, 300, rows_sf))
    assert torch.equal(q.codes.cpu()[:300], host.codes)


@gpu
@pytest.mark.parametrize("fmt", ["mxfp8", "nvfp4"])
@pytest.mark.parametrize("M,N,K,bn", [(128, 128, 256, 128), (256, 512, 1024, 128), (100, 384, 512, 128),
                                       (2048, 1024, 512, 256), (520, 256, 4096, 128), (37, 256, 2048, 256)])
def test_blockscaled_gemm_matches_fp32_of_the_same_operands(fmt, M, N, K, bn):
    dev = torch.device("cuda")
    torch.manual_seed(M + N + K)
    a = bs.quantize(torch.randn(M, K) * torch.logspace(-1, 1, M)[:, None], fmt)
    w = bs.quantize(torch.randn(N, K) * 0.05 * torch.logspace(-1, 1, N)[:, None], fmt)
    ref = a.dequantize() @ w.dequantize().t()
    ad = bs.BlockScaled(a.fmt, M, a.k, torch.zeros((M + 255) // 256 * 256, a.codes.shape[1], dtype=torch.uint8), a.sf, a.tensor_scale)
    ad.codes[:M] = a.codes
    pad_sf = torch.zeros(bs.sf_bytes((M + 255) // 256 * 256, a.k // a.vec), dtype=torch.uint8)
    pad_sf[:a.sf.numel()] = a.sf
    ad.sf = pad_sf
    got = bs.gemm(ad.to(dev), w.to(dev), out_dtype=torch.float32, bn=bn)
    _rows_close(got, ref, 2e-3)
    bias = torch.randn(N)
    got = bs.gemm(ad.to(dev), w.to(dev), bias=bias.to(dev), bn=bn)
    _rows_close(got, ref + bias, 1e-2)


@gpu
@pytest.mark.parametrize("fmt", ["mxfp8", "nvfp4"])
def test_blockscaled_epilogues_and_grouped(fmt):
    dev = torch.device("cuda")
    torch.manual_seed(11)
    M, H, I = 256, 512, 768
    x = (torch.randn(M, H) * 2.0).to(torch.bfloat16)
    xq = bs.quantize_act(x.to(dev), fmt, tensor_scale=0.02)
    xh = bs.BlockScaled(xq.fmt, M, H, xq.codes.cpu()[:M], xq.sf.cpu(), xq.tensor_scale)
    # residual + row statistics
    wo = bs.quantize(torch.randn(H, H) * 0.05, fmt)
    res = torch.randn(M, H).to(torch.bfloat16)
    want, want_ss = bs.gemm_residual(xh, wo, res)
    got, ss = bs.gemm_residual(xq, wo.to(dev), res.to(dev))
    _rows_close(got, want)
    torch.testing.assert_close(ss.sum(-1).cpu(), want.float().pow(2).sum(-1), rtol=2e-2, atol=1e-2)
    # gate/up with the RMSNorm row scale and SwiGLU
    gu = L.interleave_gate_up(torch.randn(I, H) * 0.05, torch.randn(I, H) * 0.05)
    wgu = bs.quantize(gu, fmt)
    row_ss = x.float().pow(2).sum(-1, keepdim=True)
    want = bs.gemm_glu(xh, wgu, act=0, row_ss=row_ss, norm_dim=H, eps=1e-6)
    got = bs.gemm_glu(xq, wgu.to(dev), act=0, row_ss=row_ss.to(dev), norm_dim=H, eps=1e-6)
    _rows_close(got, want)
    # grouped (MoE): 128-row blocks pick their expert; an inactive block is skipped
    E, N = 4, 256
    wst = bs.quantize(torch.randn(E * N, H) * 0.05, fmt)
    grp = torch.tensor([2, -1], dtype=torch.int32)
    want = bs.gemm(xh, wst, mblk_group=grp, num_groups=E)
    out = torch.zeros(M, N, dtype=torch.bfloat16, device=dev)
    got = bs.gemm(xq, wst.to(dev), out=out, mblk_group=grp.to(dev), num_groups=E)
    _rows_close(got[:128], want[:128])
    assert float(got[128:].abs().max()) == 0.0


@gpu
@pytest.mark.parametrize("fmt", ["mxfp8", "nvfp4"])
def test_blockscaled_qkv_epilogue(fmt):
    dev = torch.device("cuda")
    torch.manual_seed(5)
    M, H, n_q, n_kv = 200, 512, 4, 2
    x = torch.randn(M, H).to(torch.bfloat16)
    xq = bs.quantize_act(x.to(dev), fmt, tensor_scale=0.02)
    xh = bs.BlockScaled(xq.fmt, M, H, xq.codes.cpu()[:M], xq.sf.cpu(), xq.tensor_scale)
    w = bs.quantize(torch.randn((n_q + 2 * n_kv) * 128, H) * 0.05, fmt)
    pos = torch.arange(M, dtype=torch.int32)
    slots = torch.arange(M, dtype=torch.int32) + 16
    cos = torch.cos(torch.arange(512)[:, None] * torch.logspace(0, -3, 64)[None]).float().contiguous()
    sin = torch.sin(torch.arange(512)[:, None] * torch.logspace(0, -3, 64)[None]).float().contiguous()
    qn, kn = torch.rand(128) + 0.5, torch.rand(128) + 0.5
    row_ss = x.float().pow(2).sum(-1, keepdim=True)
    outs = {}
    for name, d, a, ww in (("cpu", "cpu", xh, w), ("gpu", dev, xq, w.to(dev))):
        q_out = torch.zeros(M, n_q * 128, dtype=torch.bfloat16, device=d)
        kv = torch.zeros(16, 2, n_kv, 16, 128, dtype=torch.bfloat16, device=d)
        bs.gemm_qkv(a, ww, n_q=n_q, n_kv=n_kv, q_out=q_out, kv_cache=kv, slot_mapping=slots.to(d), positions=pos.to(d),
                    cos_t=cos.to(d), sin_t=sin.to(d), q_norm_w=qn.to(d), k_norm_w=kn.to(d), row_ss=row_ss.to(d),
                    norm_dim=H, eps=1e-6)
        outs[name] = (q_out.cpu(), kv.cpu())
    _rows_close(outs["gpu"][0], outs["cpu"][0], 3e-2)
    _rows_close(outs["gpu"][1].reshape(-1, 128), outs["cpu"][1].reshape(-1, 128), 3e-2)


def _tiny_model(weight_quant, device, dtype):
    from gllm_b200.models.config import preset
    from gllm_b200.models.decoder import DecoderModel
    from gllm_b200.models.weights import RandomWeights
    cfg = preset("tiny-qwen3")
    src = RandomWeights(cfg, "cpu", torch.float32, seed=4, std=0.05)
    return cfg, DecoderModel(cfg, src, device=device, dtype=dtype, max_positions=256, weight_quant=weight_quant)


def _prefill_batch(cfg, T, d):
    from gllm_b200.engine.batch import ForwardBatch
    ids = (torch.arange(T, dtype=torch.int32) * 7 + 3) % cfg.vocab_size
    return ForwardBatch(token_ids=ids.to(d), positions=torch.arange(T, dtype=torch.int32, device=d),
                        slot_mapping=torch.arange(T, dtype=torch.int32, device=d),
                        block_tables=torch.arange(16, dtype=torch.int32, device=d)[None],
                        ctx_lens=torch.tensor([T], dtype=torch.int32, device=d),
                        q_start=torch.tensor([0], dtype=torch.int32, device=d),
                        q_len=torch.tensor([T], dtype=torch.int32, device=d), max_q_len=T)


@pytest.mark.parametrize("fmt", ["mxfp8", "nvfp4"])
def test_decoder_with_block_scaled_weights_tracks_the_unquantised_model_on_cpu(fmt):
    cfg, ref = _tiny_model(None, "cpu", torch.float32)
    _, q = _tiny_model(fmt, "cpu", torch.float32)
    assert q.bs_fmt == fmt and q.weight_bytes() < 0.6 * ref.weight_bytes()
    want = ref.forward(_prefill_batch(cfg, 45, "cpu"), ref.alloc_kv_cache(16))[:, :cfg.vocab_size]
    got = q.forward(_prefill_batch(cfg, 45, "cpu"), q.alloc_kv_cache(16))[:, :cfg.vocab_size]
    cos = torch.nn.functional.cosine_similarity(got.flatten(), want.flatten(), dim=0).item()
    assert cos > (0.985 if fmt == "mxfp8" else 0.85), cos


@gpu
@pytest.mark.parametrize("fmt", ["mxfp8", "nvfp4"])
def test_decoder_with_block_scaled_weights_gpu_matches_cpu_oracle(fmt):
    """The fused layer (QKV / GLU / residual epilogues) on block-scaled tensor cores against the same model on the
    CPU oracle: same quantised weights, activations quantised by the same rule."""
    cfg, cpu = _tiny_model(fmt, "cpu", torch.bfloat16)
    _, dev_m = _tiny_model(fmt, "cuda", torch.bfloat16)
    assert dev_m.fused and dev_m.bs_fmt == fmt
    want = cpu.forward(_prefill_batch(cfg, 150, "cpu"), cpu.alloc_kv_cache(16))[:, :cfg.vocab_size].float()
    got = dev_m.forward(_prefill_batch(cfg, 150, "cuda"), dev_m.alloc_kv_cache(16))[:, :cfg.vocab_size].float().cpu()
    cos = torch.nn.functional.cosine_similarity(got.flatten(), want.flatten(), dim=0).item()
    # 4-bit activations: a bf16 rounding difference upstream flips codes downstream, so the two models drift apart more
    assert cos > (0.99 if fmt == "mxfp8" else 0.95), cos


def _tiny_moe(expert_quant, device, dtype):
    from gllm_b200.models.config import preset
    from gllm_b200.models.decoder import DecoderModel
    from gllm_b200.models.weights import RandomWeights
    cfg = preset("tiny-moe")
    cfg.moe_intermediate_size = 256
    cfg.num_shared_experts = 1
    src = RandomWeights(cfg, "cpu", torch.float32, seed=6, std=0.05)
    return cfg, DecoderModel(cfg, src, device=device, dtype=dtype, max_positions=256, expert_quant=expert_quant,
                             fused=True)


@pytest.mark.parametrize("fmt", ["mxfp8", "nvfp4"])
def test_moe_with_block_scaled_experts_tracks_the_unquantised_model_on_cpu(fmt):
    """MXFP8 / NVFP4 expert stacks with bf16 attention (the Qwen3-30B-A3B configuration of the benchmarks)."""
    cfg, ref = _tiny_moe(None, "cpu", torch.float32)
    _, q = _tiny_moe(fmt, "cpu", torch.float32)
    assert q.layers[0].moe.bs_fmt == fmt and isinstance(q.layers[0].wqkv, torch.Tensor)
    want = ref.forward(_prefill_batch(cfg, 45, "cpu"), ref.alloc_kv_cache(16))[:, :cfg.vocab_size]
    got = q.forward(_prefill_batch(cfg, 45, "cpu"), q.alloc_kv_cache(16))[:, :cfg.vocab_size]
    cos = torch.nn.functional.cosine_similarity(got.flatten(), want.flatten(), dim=0).item()
    assert cos > (0.99 if fmt == "mxfp8" else 0.9), cos


@gpu
@pytest.mark.parametrize("fmt", ["mxfp8", "nvfp4"])
def test_moe_with_block_scaled_experts_gpu_matches_cpu_oracle(fmt):
    cfg, cpu = _tiny_moe(fmt, "cpu", torch.bfloat16)
    _, dev_m = _tiny_moe(fmt, "cuda", torch.bfloat16)
    want = cpu.forward(_prefill_batch(cfg, 150, "cpu"), cpu.alloc_kv_cache(16))[:, :cfg.vocab_size].float()
    got = dev_m.forward(_prefill_batch(cfg, 150, "cuda"), dev_m.alloc_kv_cache(16))[:, :cfg.vocab_size].float().cpu()
    cos = torch.nn.functional.cosine_similarity(got.flatten(), want.flatten(), dim=0).item()
    # 4-bit activations: a bf16 rounding difference upstream flips codes downstream, so the two models drift apart more
    assert cos > (0.99 if fmt == "mxfp8" else 0.95), cos
