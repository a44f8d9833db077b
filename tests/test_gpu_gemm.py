"""tcgen05 GEMM family vs an fp32 PyTorch reference of the same op (run with -m gpu on a B200)."""
import pytest
import torch

from gllm_b200 import ops
from gllm_b200.ops import linear as L

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _rand(*shape, scale=1.0):
    return (torch.randn(*shape, device=DEV) * scale).to(torch.bfloat16)


def _close(got, ref, tol=2e-2):
    got, ref = got.float(), ref.float()
    err = (got - ref).abs().max().item()
    denom = ref.abs().max().item() + 1e-6
    assert err / denom < tol, f"max abs err {err} vs ref max {denom}"
    cos = torch.nn.functional.cosine_similarity(got.flatten(), ref.flatten(), dim=0).item()
    assert cos > 0.9995, f"cosine {cos}"
    # row by row: an error confined to a few rows or one tile column must not hide behind the global maximum
    g2, r2 = got.reshape(-1, got.shape[-1]), ref.reshape(-1, ref.shape[-1])
    row_err = (g2 - r2).abs().amax(-1)
    row_ref = r2.abs().amax(-1)
    bad = (row_err > 2 * tol * row_ref + 0.002 * denom).nonzero().flatten()
    assert bad.numel() == 0, f"rows {bad[:8].tolist()} off by {row_err[bad[:8]].tolist()} (row max {row_ref[bad[:8]].tolist()})"


@pytest.mark.parametrize("M,N,K,bn", [
    (128, 128, 64, 128), (128, 256, 64, 256), (256, 4096, 4096, 256), (256, 4096, 4096, 128),
    (100, 384, 192, 128), (1, 128, 64, 128), (300, 1024, 520, 256), (777, 2176, 1000, 128),
    (2048, 6144, 4096, 128), (129, 32, 4096, 128),
])
def test_gemm_plain(M, N, K, bn):
    torch.manual_seed(0)
    a, w = _rand(M, K), _rand(N, K, scale=0.05)
    out = ops.gemm(a, w, bn=bn)
    _close(out, a.float() @ w.float().t())


def test_gemm_softcap_epilogue_and_narrow_tiles():
    """Final-logit soft cap inside the store epilogue (fp32 logits, fused norm scale), and the 64-wide residual tiles."""
    torch.manual_seed(3)
    M, N, K = 200, 2048, 1024
    a, w = _rand(M, K), _rand(N, K, scale=0.2)
    ss = a.float().pow(2).sum(-1, keepdim=True).contiguous()
    out = ops.gemm(a, w, out_dtype=torch.float32, row_ss=ss, norm_dim=K, eps=1e-6, bn=256, softcap=30.0)
    x = (a.float() * torch.rsqrt(ss / K + 1e-6)) @ w.float().t()
    ref = torch.tanh(x / 30.0) * 30.0
    assert x.abs().max() > 20.0          # the cap actually bends some values
    _close(out, ref)
    r = _rand(M, N)
    o, ss_out = ops.gemm_residual(a, w, r, bn=64)
    want = (a.float() @ w.float().t() + r.float())
    _close(o, want)
    torch.testing.assert_close(ss_out[:M, :N // 64].sum(-1), o.float().pow(2).sum(-1), rtol=2e-3, atol=2e-3)


@pytest.mark.parametrize("M,N,K,bn,splits", [
    (256, 4096, 4096, 256, 9), (256, 4096, 12288, 256, 16), (100, 512, 1024, 128, 4), (256, 6144, 4096, 128, 3),
    (200, 768, 2048, 256, 2), (512, 1024, 1024, 256, 5), (256, 4096, 4096, 256, 0),
])
def test_gemm_split_k(M, N, K, bn, splits):
    """Split-K with in-kernel ticket reduction: same answer as one pass, bit-identical across launches."""
    torch.manual_seed(8)
    a, w = _rand(M, K), _rand(N, K, scale=0.05)
    out = ops.gemm(a, w, bn=bn, splits=splits).clone()
    _close(out, a.float() @ w.float().t())
    assert torch.equal(out, ops.gemm(a, w, bn=bn, splits=splits))
    r = _rand(M, N)
    o2, ss = ops.gemm_residual(a, w, r, bn=bn, splits=splits)
    _close(o2, a.float() @ w.float().t() + r.float())
    torch.testing.assert_close(ss.sum(-1), o2.float().pow(2).sum(-1), rtol=1e-3, atol=1e-3)


def test_gemm_fp32_out_bias_rowscale():
    torch.manual_seed(1)
    M, N, K = 200, 512, 1024
    a, w = _rand(M, K), _rand(N, K, scale=0.05)
    bias = torch.randn(N, device=DEV)
    ss = a.float().pow(2).sum(-1, keepdim=True).contiguous()
    out = ops.gemm(a, w, out_dtype=torch.float32, bias=bias, row_ss=ss, norm_dim=K, eps=1e-6, bn=128)
    ref = (a.float() @ w.float().t()) * torch.rsqrt(ss / K + 1e-6) + bias
    _close(out, ref, 5e-3)


@pytest.mark.parametrize("M,N,K,bn", [(256, 4096, 4096, 256), (100, 1024, 512, 128), (300, 4096, 1536, 128)])
def test_gemm_residual(M, N, K, bn):
    torch.manual_seed(2)
    a, w, r = _rand(M, K), _rand(N, K, scale=0.05), _rand(M, N)
    out, ss = ops.gemm_residual(a, w, r, bn=bn)
    ref = (a.float() @ w.float().t() + r.float())
    _close(out, ref)
    ss_ref = out.float().pow(2).sum(-1)
    torch.testing.assert_close(ss.sum(-1), ss_ref, rtol=1e-3, atol=1e-3)


@pytest.mark.parametrize("splits", [0, 1, 3])
@pytest.mark.parametrize("M,I,K,bn,act", [(256, 1024, 512, 256, 0), (100, 768, 2048, 128, 0), (64, 512, 256, 256, 1),
                                          (256, 12288, 4096, 256, 0), (256, 1536, 1024, 192, 0),
                                          (100, 960, 512, 192, 1), (2048, 1024, 512, 256, 0), (300, 1536, 1024, 128, 0)])
def test_gemm_glu(M, I, K, bn, act, splits):
    torch.manual_seed(3)
    a, g, u = _rand(M, K), _rand(I, K, scale=0.05), _rand(I, K, scale=0.05)
    ss = a.float().pow(2).sum(-1, keepdim=True).contiguous()
    wp = ops.interleave_gate_up(g, u, bn)
    out = ops.gemm_glu(a, wp, act=act, row_ss=ss, norm_dim=K, eps=1e-5, bn=bn, splits=splits)
    rs = torch.rsqrt(ss / K + 1e-5)
    gv, uv = (a.float() @ g.float().t()) * rs, (a.float() @ u.float().t()) * rs
    actf = torch.nn.functional.silu if act == 0 else (lambda x: torch.nn.functional.gelu(x, approximate="tanh"))
    _close(out, actf(gv) * uv)


def test_gemm_grouped_and_glu_grouped():
    torch.manual_seed(4)
    E, N, K = 4, 512, 256
    mblk = torch.tensor([2, 0, 3, 3, 1], dtype=torch.int32, device=DEV)
    M = 128 * mblk.numel()
    a, w = _rand(M, K), _rand(E * N, K, scale=0.05)
    out = ops.gemm_grouped(a, w, mblk, E, bn=128)
    ref = torch.cat([a[i * 128:(i + 1) * 128].float() @ w[int(e) * N:(int(e) + 1) * N].float().t()
                     for i, e in enumerate(mblk.tolist())])
    _close(out, ref)
    out2 = ops.gemm_glu(a, w, act=0, bn=128, mblk_group=mblk, num_groups=E)
    ref2 = L.gemm_glu(a.cpu(), w.cpu(), act=0, bn=128, mblk_group=mblk.cpu(), num_groups=E)
    _close(out2, ref2.to(DEV))


@pytest.mark.parametrize("M,splits", [(150, 0), (150, 1), (256, 3), (64, 4), (700, 0)])
@pytest.mark.parametrize("qk_norm", [True, False])
def test_gemm_qkv_fused(qk_norm, M, splits):
    torch.manual_seed(5)
    K, n_q, n_kv, D = 1024, 8, 2, 128
    pages, max_pos = 64, 512
    a = _rand(M, K)
    w = _rand((n_q + 2 * n_kv) * D, K, scale=0.05)
    ss = a.float().pow(2).sum(-1, keepdim=True).contiguous()
    qn = (torch.rand(D, device=DEV) + 0.5) if qk_norm else None
    kn = (torch.rand(D, device=DEV) + 0.5) if qk_norm else None
    inv = 1.0 / (10000.0 ** (torch.arange(0, D, 2, device=DEV).double() / D))
    ang = torch.arange(max_pos, device=DEV).double()[:, None] * inv[None]
    cos_t, sin_t = ang.cos().float().contiguous(), ang.sin().float().contiguous()
    positions = torch.randint(0, max_pos, (M,), device=DEV, dtype=torch.int32)
    slots = torch.randperm(pages * 16, device=DEV)[:M].to(torch.int32)
    slots[3] = -1
    kv = torch.zeros(pages, 2, n_kv, 16, D, device=DEV, dtype=torch.bfloat16)
    q_out = torch.zeros(M, n_q * D, device=DEV, dtype=torch.bfloat16)
    ops.gemm_qkv(a, w, n_q=n_q, n_kv=n_kv, q_out=q_out, kv_cache=kv, slot_mapping=slots, positions=positions,
                 cos_t=cos_t, sin_t=sin_t, q_norm_w=qn, k_norm_w=kn, qk_eps=1e-6, row_ss=ss, norm_dim=K, eps=1e-6,
                 splits=splits)
    acc = (a.float() @ w.float().t()) * torch.rsqrt(ss / K + 1e-6)
    q, k, v = L.qkv_post_ref(acc, n_q, n_kv, D, positions, cos_t, sin_t, qn, kn, 1e-6)
    _close(q_out, q.reshape(M, -1))
    kv_ref = torch.zeros_like(kv)
    L.kv_write_ref(kv_ref, k, v, slots)
    _close(kv, kv_ref)


def test_gemm_fp8():
    torch.manual_seed(6)
    M, N, K = 256, 512, 1024
    a = (torch.randn(M, K, device=DEV)).to(torch.float8_e4m3fn)
    w = (torch.randn(N, K, device=DEV) * 0.5).to(torch.float8_e4m3fn)
    sa = torch.rand(M, device=DEV) + 0.5
    sb = torch.rand(N, device=DEV) + 0.5
    out = ops.gemm_fp8(a, w, sa, sb, bn=128)
    ref = (a.float() @ w.float().t()) * sa[:, None] * sb[None, :]
    _close(out, ref)


def test_gemm_determinism_and_reuse():
    """Same launch twice must be bit-identical (catches races in the barrier protocol)."""
    torch.manual_seed(7)
    a, w = _rand(512, 2048), _rand(4096, 2048, scale=0.05)
    o1 = ops.gemm(a, w).clone()
    for _ in range(3):
        o2 = ops.gemm(a, w)
    assert torch.equal(o1, o2)


@pytest.fixture
def cta_pairs():
    """Route 128 < M <= 256 through the CTA-pair kernels (tcgen05.mma.cta_group::2) for the duration of a test."""
    old = ops.set_pair_max_m(256, 0xF)
    try:
        yield
    finally:
        ops.set_pair_max_m(*old)


def test_cta_pair_kernels_match_reference(cta_pairs):
    """Every fused epilogue on the CTA-pair path: the existing cases whose M falls in the pair range."""
    for M, N, K, bn in [(256, 4096, 4096, 256), (256, 4096, 4096, 128), (129, 32, 4096, 128), (200, 384, 520, 128)]:
        test_gemm_plain(M, N, K, bn)
    for M, N, K, bn, sp in [(256, 4096, 4096, 256, 9), (256, 4096, 12288, 256, 4), (256, 6144, 4096, 128, 3),
                            (200, 768, 2048, 256, 2), (256, 4096, 4096, 128, 0)]:
        test_gemm_split_k(M, N, K, bn, sp)
    test_gemm_residual(256, 4096, 4096, 256)
    test_gemm_residual(150, 1024, 512, 128)
    for M, I, K, bn, act in [(256, 1024, 512, 256, 0), (256, 12288, 4096, 256, 0), (256, 1536, 1024, 192, 0),
                             (130, 960, 512, 192, 1), (256, 1536, 1024, 128, 0)]:
        for sp in (0, 1, 3):
            test_gemm_glu(M, I, K, bn, act, sp)
    for qk_norm in (True, False):
        for M, sp in [(150, 0), (256, 3), (256, 1)]:
            test_gemm_qkv_fused(qk_norm, M, sp)


def test_cta_pair_kernels_are_deterministic(cta_pairs):
    torch.manual_seed(11)
    a, w, r = _rand(256, 4096), _rand(4096, 4096, scale=0.05), _rand(256, 4096)
    o1, s1 = ops.gemm_residual(a, w, r, bn=128)
    o1, s1 = o1.clone(), s1.clone()
    for _ in range(3):
        o2, s2 = ops.gemm_residual(a, w, r, bn=128)
    assert torch.equal(o1, o2) and torch.equal(s1, s2)


def test_large_m_kernels_with_and_without_cta_pairs():
    """256-wide tiles at prefill sizes: the CTA-pair kernels (default) and the single-CTA kernels give the same answer."""
    for big in (1024, 0):
        old = ops.set_pair_big_m(big)
        try:
            test_gemm_plain(2048, 4096, 1024, 256)
            test_gemm_plain(1100, 768, 520, 256)
            test_gemm_residual(2048, 4096, 1536, 256)
            test_gemm_glu(2048, 1024, 512, 256, 0, 0)
            test_gemm_glu(3000, 1536, 1024, 256, 1, 0)
        finally:
            ops.set_pair_big_m(old)


@pytest.mark.parametrize("M,splits", [(150, 0), (256, 3), (700, 0)])
def test_gemm_qkv_fused_fp8_kv_cache(M, splits):
    """The fused QKV epilogue writing an fp8 (e4m3) paged cache: value / kv_scale, saturating."""
    torch.manual_seed(15)
    K, n_q, n_kv, D = 1024, 8, 2, 128
    pages, max_pos, kv_scale = 64, 512, 0.125
    a = _rand(M, K)
    w = _rand((n_q + 2 * n_kv) * D, K, scale=0.05)
    ss = a.float().pow(2).sum(-1, keepdim=True).contiguous()
    qn, kn = torch.rand(D, device=DEV) + 0.5, torch.rand(D, device=DEV) + 0.5
    inv = 1.0 / (10000.0 ** (torch.arange(0, D, 2, device=DEV).double() / D))
    ang = torch.arange(max_pos, device=DEV).double()[:, None] * inv[None]
    cos_t, sin_t = ang.cos().float().contiguous(), ang.sin().float().contiguous()
    positions = torch.randint(0, max_pos, (M,), device=DEV, dtype=torch.int32)
    slots = torch.randperm(pages * 16, device=DEV)[:M].to(torch.int32)
    slots[3] = -1
    kv = torch.zeros(pages, 2, n_kv, 16, D, device=DEV, dtype=torch.uint8).view(torch.float8_e4m3fn)
    q_out = torch.zeros(M, n_q * D, device=DEV, dtype=torch.bfloat16)
    ops.gemm_qkv(a, w, n_q=n_q, n_kv=n_kv, q_out=q_out, kv_cache=kv, slot_mapping=slots, positions=positions,
                 cos_t=cos_t, sin_t=sin_t, q_norm_w=qn, k_norm_w=kn, qk_eps=1e-6, row_ss=ss, norm_dim=K, eps=1e-6,
                 splits=splits, kv_scale=kv_scale)
    acc = (a.float() @ w.float().t()) * torch.rsqrt(ss / K + 1e-6)
    q, k, v = L.qkv_post_ref(acc, n_q, n_kv, D, positions, cos_t, sin_t, qn, kn, 1e-6)
    _close(q_out, q.reshape(M, -1))
    kv_ref = torch.zeros_like(kv)
    L.kv_write_ref(kv_ref, k, v, slots, kv_scale)
    got, ref = kv.float() * kv_scale, kv_ref.float() * kv_scale
    assert (got - ref).abs().max().item() <= 0.13 * ref.abs().max().item()      # at most one e4m3 step apart
    assert torch.nn.functional.cosine_similarity(got.flatten(), ref.flatten(), dim=0).item() > 0.999


def test_split_k_gemms_on_two_streams_with_their_own_workspaces():
    """A stream with its own split-K scratch and barrier words: split-K GEMMs launched on it overlap GEMMs of the default
    workspace (another stream) and both give the right result, many times over."""
    from gllm_b200.ops import _native as nv
    torch.manual_seed(5)
    M, N, K = 256, 4096, 4096
    a1, w1 = _rand(M, K), _rand(N, K, scale=0.05)
    a2, w2 = _rand(M, K), _rand(N, K, scale=0.05)
    ref1, ref2 = a1.float() @ w1.float().t(), a2.float() @ w2.float().t()
    s1, s2 = torch.cuda.Stream(), torch.cuda.Stream()
    nv.stream_splitk_workspace(s1)
    o1 = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
    o2 = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
    torch.cuda.synchronize()
    for _ in range(20):
        with torch.cuda.stream(s1):
            ops.gemm(a1, w1, out=o1, bn=128, splits=4)
        with torch.cuda.stream(s2):
            ops.gemm(a2, w2, out=o2, bn=128, splits=4)
    torch.cuda.synchronize()
    _close(o1, ref1)
    _close(o2, ref2)
    assert nv.device_error() == 0
