import numpy as np
import torch

from gllm_b200.kv_cache import (KV_PAGE_HEADER_DTYPE, CompressionCodec, DoubleBufferedKvState, DualTrackPool, HardwareProfile,
                                KvDecisionMatrix, KvPageHeaderTable, KvPageLayout, KvVariant, PrecisionTier, StorageTier,
                                TurboQuantConfig, TurboQuantRuntime, fwht, kivi_dequantize, stochastic_round)
from gllm_b200.kv_cache.quant import (fp8_dequantize_page, fp8_quantize_page, kivi_quantize_page, pack_codes, unpack_codes)


def test_header_is_64_bytes_and_round_trips():
    assert KV_PAGE_HEADER_DTYPE.itemsize == 64
    t = KvPageHeaderTable(8)
    t.bind(3, sequence_id=(7 << 32) | 5, logical_index=9, now=100, pipeline=1)
    t.record_telemetry(3, entropy=2.5, softmax_max=0.9, delta_rho=0.25, dead_ratio=0.5, head_spread=300)
    t.age_all(); t.age_all(); t.touch(2, 101)
    raw = t.as_bytes()
    assert len(raw) == 8 * 64
    back = np.frombuffer(raw, dtype=KV_PAGE_HEADER_DTYPE)
    assert back[3]["sequence_id"] == (7 << 32) | 5 and back[3]["logical_index"] == 9 and back[3]["head_spread"] == 255
    assert back[3]["tier_age"] == 2 and back[2]["tier_age"] == 0 and abs(float(back[3]["entropy"]) - 2.5) < 1e-3
    assert back[3]["precision_tier"] == PrecisionTier.FP16 and back[3]["storage_tier"] == StorageTier.HBM
    assert CompressionCodec.ZSTD == 2 and PrecisionTier.KIVI2.bits == 2


def test_page_layout_matches_pool_addressing():
    lay = KvPageLayout(num_layers=36, num_kv_heads=8, head_dim=128)
    assert lay.layer_stride == 2 * 8 * 16 * 128 * 2 and lay.page_stride == 36 * lay.layer_stride
    assert lay.v_offset(0, 0, 0) - lay.k_offset(0, 0, 0) == 8 * 16 * 128 * 2
    assert lay.k_offset(2, 3, 5) == 2 * lay.layer_stride + (3 * 16 + 5) * 128 * 2
    assert lay.bytes_per_token() == 36 * 2 * 8 * 128 * 2 and lay.pages_for(17) == 2
    mla = KvPageLayout(num_layers=61, num_kv_heads=1, head_dim=0, mla_dim=576)
    assert mla.page_stride == 61 * 16 * 576 * 2 and mla.k_offset(1, 0, 2) == mla.layer_stride + 2 * 576 * 2
    db = DoubleBufferedKvState()
    db.stage(1, "a"); assert db.get(1) is None
    db.publish(); assert db.get(1) == "a" and db.generation == 1


def test_fwht_kivi_fp8_and_packing():
    torch.manual_seed(0)
    x = torch.randn(16, 128)
    torch.testing.assert_close(fwht(fwht(x)), x, rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(fwht(x).pow(2).sum(), x.pow(2).sum(), rtol=1e-4, atol=1e-3)     # orthonormal
    k = torch.randn(16, 128); k[:, 7] *= 30                      # an outlier channel
    v = torch.randn(16, 128)
    for bits, tol in ((4, 0.12), (2, 0.6)):
        p = kivi_quantize_page(k, v, bits=bits)
        kd, vd = kivi_dequantize(p)
        assert ((kd - k).abs() / k.abs().amax(0, keepdim=True)).max() < tol      # per-channel scaling holds outliers
        assert (vd - v).abs().max() < tol * v.abs().max() * 1.2
        assert p.k_q.max() < 2 ** bits
    pr = kivi_quantize_page(k, v, bits=4, rotate=True)
    kd, _ = kivi_dequantize(pr)
    assert (kd - k).pow(2).mean().sqrt() < 0.5
    codes = torch.randint(0, 4, (5, 64), dtype=torch.uint8)
    assert torch.equal(unpack_codes(pack_codes(codes, 2), 2), codes) and pack_codes(codes, 2).shape == (5, 16)
    g = torch.Generator().manual_seed(1)
    xs = torch.full((20000,), 0.3)
    assert abs(stochastic_round(xs, g).mean().item() - 0.3) < 0.02
    q, s = fp8_quantize_page(k)
    assert (fp8_dequantize_page(q, s, torch.float32) - k).abs().max() < 0.07 * k.abs().max()


def test_turboquant_sinks_and_dual_track():
    torch.manual_seed(1)
    k, v = torch.randn(16, 64), torch.randn(16, 64)
    assert not TurboQuantConfig.default_for(False).enabled
    rt = TurboQuantRuntime(TurboQuantConfig.default_for(True))
    assert rt.cfg.bits == 4 and rt.cfg.sink_tokens == 4 and rt.cfg.use_fwht and not rt.cfg.dual_track
    rt.compress((0, 0, 0), k, v, first_token_index=0)
    kd, vd = rt.decompress((0, 0, 0), torch.float32)
    torch.testing.assert_close(kd[:4], k[:4]); torch.testing.assert_close(vd[:4], v[:4])      # sinks exact
    assert (kd[4:] - k[4:]).abs().max() < 0.5 and rt.compression_ratio() > 1.5
    rt.compress((1, 0, 0), k, v, first_token_index=16)                                        # no sinks on later pages
    assert rt.pages[(1, 0, 0)][1] is None
    pool = DualTrackPool(main_bits=2)
    pool.put("p", k, v)
    e_main = (pool.get("p", use_residual=False)[0] - k).pow(2).mean()
    e_both = (pool.get("p")[0] - k).pow(2).mean()
    assert e_both < e_main
    assert pool.drop_residual() > 0 and "p" not in pool.residual


def test_decision_matrix():
    assert [KvVariant.from_index(i).index for i in range(16)] == list(range(16))
    dm = KvDecisionMatrix(HardwareProfile(hbm_bytes=100 << 30))
    assert dm.choose(10 << 30, 20 << 30, False, True) == KvVariant()
    v = dm.choose(200 << 30, 20 << 30, True, True)
    assert v.kivi and not v.mustafar
    assert dm.page_tier(v, 250, 0.5) == PrecisionTier.FP16 and dm.page_tier(v, 100, 0.5) == PrecisionTier.KIVI4
    assert dm.page_tier(KvVariant(True, True), 50, 0.1) == PrecisionTier.KIVI4 and dm.page_tier(KvVariant(True), 50, 0.1) == PrecisionTier.KIVI2
