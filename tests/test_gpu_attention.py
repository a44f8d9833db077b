"""Paged attention kernels vs the fp32 reference (run with -m gpu on a B200)."""
import pytest
import torch

from gllm_b200 import ops

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _setup(ctx_lens, n_kv, D, extra_pages=8, seed=0):
    torch.manual_seed(seed)
    B = len(ctx_lens)
    need = [(c + 15) // 16 for c in ctx_lens]
    total = sum(need) + extra_pages
    kv = (torch.randn(total, 2, n_kv, 16, D, device=DEV)).to(torch.bfloat16)
    perm = torch.randperm(total, device=DEV).to(torch.int32)
    max_blocks = max(need) + 2
    bt = torch.zeros(B, max_blocks, dtype=torch.int32, device=DEV)
    o = 0
    for i, n in enumerate(need):
        bt[i, :n] = perm[o:o + n]
        o += n
    return kv, bt


def _close(got, ref, tol=2e-2):
    got, ref = got.float(), ref.float()
    err = (got - ref).abs().max().item()
    assert err < tol * (ref.abs().max().item() + 1e-6), f"max err {err}"


@pytest.mark.parametrize("n_q,n_kv,pps", [(8, 2, 32), (4, 1, 4), (32, 8, 8), (16, 1, 1000)])
def test_paged_decode(n_q, n_kv, pps):
    D = 128
    ctx = [1, 16, 17, 100, 515, 2304, 33, 64]
    kv, bt = _setup(ctx, n_kv, D)
    B = len(ctx)
    q = torch.randn(B, n_q * D, device=DEV).to(torch.bfloat16)
    cl = torch.tensor(ctx, dtype=torch.int32, device=DEV)
    out = ops.paged_decode(q, kv, bt, cl, n_q=n_q, n_kv=n_kv, pages_per_split=pps)
    ar = torch.arange(B, dtype=torch.int32, device=DEV)
    ref = ops.attention_ref(q, kv, bt, ar, torch.ones_like(cl), cl, n_q, n_kv, D ** -0.5)
    _close(out, ref)
    # second launch reuses the ticket counters: must give the same answer
    out2 = ops.paged_decode(q, kv, bt, cl, n_q=n_q, n_kv=n_kv, pages_per_split=pps)
    _close(out2, ref)


def test_paged_decode_empty_slots_window_sinks():
    D, n_q, n_kv = 128, 8, 2
    ctx = [0, 300, 0, 40]
    kv, bt = _setup([max(c, 1) for c in ctx], n_kv, D, seed=1)
    q = torch.randn(4, n_q * D, device=DEV).to(torch.bfloat16)
    cl = torch.tensor(ctx, dtype=torch.int32, device=DEV)
    sinks = torch.randn(n_q, device=DEV)
    out = torch.zeros_like(q)
    ops.paged_decode(q, kv, bt, cl, n_q=n_q, n_kv=n_kv, out=out, pages_per_split=4, window=100, sinks=sinks)
    ar = torch.arange(4, dtype=torch.int32, device=DEV)
    ref = ops.attention_ref(q, kv, bt, ar, (cl > 0).int(), cl, n_q, n_kv, D ** -0.5, True, 100, sinks)
    _close(out, ref)


@pytest.mark.parametrize("n_q,n_kv", [(8, 2), (4, 4)])
def test_paged_prefill(n_q, n_kv):
    D = 128
    q_len = [5, 64, 130, 1, 257]
    ctx = [5, 200, 130, 77, 1000]   # some sequences have a cached prefix (chunked prefill / prefix reuse)
    kv, bt = _setup(ctx, n_kv, D, seed=2)
    T = sum(q_len)
    q = torch.randn(T, n_q * D, device=DEV).to(torch.bfloat16)
    qs = torch.tensor([sum(q_len[:i]) for i in range(len(q_len))], dtype=torch.int32, device=DEV)
    ql = torch.tensor(q_len, dtype=torch.int32, device=DEV)
    cl = torch.tensor(ctx, dtype=torch.int32, device=DEV)
    out = ops.paged_prefill(q, kv, bt, qs, ql, cl, max_q_len=max(q_len), n_q=n_q, n_kv=n_kv)
    ref = ops.attention_ref(q, kv, bt, qs, ql, cl, n_q, n_kv, D ** -0.5)
    _close(out, ref)
    out_b = ops.paged_prefill(q, kv, bt, qs, ql, cl, max_q_len=max(q_len), n_q=n_q, n_kv=n_kv, causal=False)
    ref_b = ops.attention_ref(q, kv, bt, qs, ql, cl, n_q, n_kv, D ** -0.5, causal=False)
    _close(out_b, ref_b)
    out_w = ops.paged_prefill(q, kv, bt, qs, ql, cl, max_q_len=max(q_len), n_q=n_q, n_kv=n_kv, window=48)
    ref_w = ops.attention_ref(q, kv, bt, qs, ql, cl, n_q, n_kv, D ** -0.5, window=48)
    _close(out_w, ref_w)


def _rows_close(got, ref, what=""):
    got, ref = got.float(), ref.float()
    row_err = (got - ref).abs().amax(-1)
    row_ref = ref.abs().amax(-1).clamp_min(1e-3)
    bad = (row_err > 0.03 * row_ref + 0.01).nonzero().flatten()
    assert bad.numel() == 0, f"{what}: rows {bad[:8].tolist()} off by {row_err[bad[:8]].tolist()}"


@pytest.mark.parametrize("n_q,n_kv", [(8, 2), (6, 2), (2, 2), (32, 8)])
def test_paged_prefill_tensor_memory_kernel(n_q, n_kv):
    """The tcgen05 prefill kernel (two query tiles per CTA: head pairs when the group size is even, row-block pairs
    otherwise) against the fp32 reference, row by row, and against the mma.sync kernel: long causal ranges, chunks
    over cached prefixes, ragged tails, sliding window, sinks."""
    from gllm_b200.ops import _native as nv
    D = 128
    q_len = [384, 1, 129, 700, 64, 256]
    ctx = [384, 300, 129, 1500, 64, 2000]
    kv, bt = _setup(ctx, n_kv, D, seed=5)
    T = sum(q_len)
    q = torch.randn(T, n_q * D, device=DEV).to(torch.bfloat16)
    qs = torch.tensor([sum(q_len[:i]) for i in range(len(q_len))], dtype=torch.int32, device=DEV)
    ql = torch.tensor(q_len, dtype=torch.int32, device=DEV)
    cl = torch.tensor(ctx, dtype=torch.int32, device=DEV)
    sinks = torch.randn(n_q, device=DEV)
    assert nv.get_option("prefill_tc") == 1
    for kw in (dict(), dict(causal=False), dict(window=100), dict(sinks=sinks), dict(window=700, sinks=sinks)):
        out = ops.paged_prefill(q, kv, bt, qs, ql, cl, max_q_len=max(q_len), n_q=n_q, n_kv=n_kv, **kw)
        ref = ops.attention_ref(q, kv, bt, qs, ql, cl, n_q, n_kv, D ** -0.5, kw.get("causal", True), kw.get("window", 0),
                                kw.get("sinks"))
        _rows_close(out.view(T * n_q, D), ref.view(T * n_q, D), f"tensor-memory kernel {kw.keys()}")
        nv.set_option("prefill_tc", 0)
        try:
            old = ops.paged_prefill(q, kv, bt, qs, ql, cl, max_q_len=max(q_len), n_q=n_q, n_kv=n_kv, **kw)
        finally:
            nv.set_option("prefill_tc", 1)
        _rows_close(out.view(T * n_q, D), old.view(T * n_q, D), f"vs mma.sync kernel {kw.keys()}")
    assert nv.device_error() == 0


def test_generic_attention_head_dim_64():
    D, n_q, n_kv = 64, 9, 3
    q_len, ctx = [7, 33], [7, 50]
    kv, bt = _setup(ctx, n_kv, D, seed=3)
    q = torch.randn(sum(q_len), n_q * D, device=DEV).to(torch.bfloat16)
    qs = torch.tensor([0, 7], dtype=torch.int32, device=DEV)
    ql = torch.tensor(q_len, dtype=torch.int32, device=DEV)
    cl = torch.tensor(ctx, dtype=torch.int32, device=DEV)
    out = ops.paged_prefill(q, kv, bt, qs, ql, cl, max_q_len=33, n_q=n_q, n_kv=n_kv)
    ref = ops.attention_ref(q, kv, bt, qs, ql, cl, n_q, n_kv, D ** -0.5)
    _close(out, ref)


def _fp8_cache(kv, scale):
    """bf16 cache -> (fp8 cache, its dequantised fp32 values)."""
    kv8 = (kv.float() / scale).clamp(-448, 448).to(torch.float8_e4m3fn)
    return kv8, kv8.float() * scale


@pytest.mark.parametrize("n_q,n_kv,pps", [(8, 2, 32), (4, 1, 4), (32, 8, 8), (16, 1, 1000)])
def test_paged_decode_fp8_cache(n_q, n_kv, pps):
    """The TMA / tensor-core decode kernel over fp8 pages (fragments converted in registers) vs the reference run on the
    dequantised cache."""
    D = 128
    ctx = [1, 16, 17, 100, 515, 2304, 33, 64]
    kv, bt = _setup(ctx, n_kv, D, seed=3)
    kv8, deq = _fp8_cache(kv, 0.05)
    B = len(ctx)
    q = torch.randn(B, n_q * D, device=DEV).to(torch.bfloat16)
    cl = torch.tensor(ctx, dtype=torch.int32, device=DEV)
    out = ops.paged_decode(q, kv8, bt, cl, n_q=n_q, n_kv=n_kv, pages_per_split=pps, kv_scale=0.05)
    ar = torch.arange(B, dtype=torch.int32, device=DEV)
    ref = ops.attention_ref(q, deq, bt, ar, torch.ones_like(cl), cl, n_q, n_kv, D ** -0.5)
    _close(out, ref)
    out2 = ops.paged_decode(q, kv8, bt, cl, n_q=n_q, n_kv=n_kv, pages_per_split=pps, kv_scale=0.05)
    _close(out2, ref)


@pytest.mark.parametrize("n_q,n_kv", [(8, 2), (4, 4)])
def test_paged_prefill_fp8_cache(n_q, n_kv):
    D = 128
    ctx = [70, 200, 16, 333]
    qlen = [70, 64, 16, 100]        # sequences 1 and 3 are later chunks over cached tokens
    kv, bt = _setup(ctx, n_kv, D, seed=4)
    kv8, deq = _fp8_cache(kv, 0.05)
    T = sum(qlen)
    q = torch.randn(T, n_q * D, device=DEV).to(torch.bfloat16)
    qs = torch.tensor([0, 70, 134, 150], dtype=torch.int32, device=DEV)
    ql = torch.tensor(qlen, dtype=torch.int32, device=DEV)
    cl = torch.tensor(ctx, dtype=torch.int32, device=DEV)
    out = ops.paged_prefill(q, kv8, bt, qs, ql, cl, max_q_len=max(qlen), n_q=n_q, n_kv=n_kv, kv_scale=0.05)
    ref = ops.attention_ref(q, deq, bt, qs, ql, cl, n_q, n_kv, D ** -0.5)
    _close(out, ref)
