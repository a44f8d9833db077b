"""The allocation-free decode-attention entry point, called through its exported C symbol.

Some callers cannot allocate device memory when they need attention (a fixed start-up memory plan, a
thread where the owning framework forbids allocator calls, a latency-critical loop), so ``gllm_paged_decode_noalloc`` keeps its
split-KV scratch in a static device array inside the library. This test loads the shared object with
ctypes, calls the symbol directly, and checks its output against the regular entry point
(``gllm_paged_decode`` with caller-provided scratch) on two calls in a row: the second call reuses a
scratch that still holds the first call's partial results.

The file name sorts last on purpose: a run that stops at the first failure has then already run every
other test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _load():
    from gllm_b200.ops import _native as nv
    lib = ctypes.CDLL(str(nv.lib_path()))
    fn = lib.gllm_paged_decode_noalloc
    P, I, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    fn.restype = I
    fn.argtypes = [P, P, P, I, P, I, P, I, I, I, F, I, I, I, P, P]
    lib.gllm_last_error.restype = ctypes.c_char_p
    lib.gllm_paged_decode_noalloc_status.restype = I
    lib.gllm_paged_decode_noalloc_status.argtypes = [P]
    return lib, fn


def _status(lib):
    """The path's own status word (read-and-clear; waits for the stream)."""
    return lib.gllm_paged_decode_noalloc_status(torch.cuda.current_stream().cuda_stream)


def _case(seed, ctx, n_q, n_kv, dev):
    torch.manual_seed(seed)
    need = [(c + 15) // 16 for c in ctx]
    total = sum(need) + 4
    kv = torch.randn(total, 2, n_kv, 16, 128, device=dev).to(torch.bfloat16)
    perm = torch.randperm(total, device=dev).to(torch.int32)
    bt = torch.zeros(len(ctx), max(need) + 1, dtype=torch.int32, device=dev)
    o = 0
    for i, n in enumerate(need):
        bt[i, :n] = perm[o:o + n]
        o += n
    q = torch.randn(len(ctx), n_q * 128, device=dev).to(torch.bfloat16)
    cl = torch.tensor(ctx, dtype=torch.int32, device=dev)
    return q, kv, bt, cl


def test_noalloc_decode_matches_regular_entry_point_twice():
    from gllm_b200 import ops
    dev = torch.device("cuda")
    lib, fn = _load()
    n_q, n_kv, pps = 8, 2, 4
    for call, ctx in enumerate([[300, 17, 1, 640, 0, 95], [33, 512, 129, 64, 700, 2]]):
        q, kv, bt, cl = _case(100 + call, [max(c, 1) for c in ctx], n_q, n_kv, dev)
        cl = torch.tensor(ctx, dtype=torch.int32, device=dev)
        max_splits = (bt.shape[1] + pps - 1) // pps
        out = torch.zeros_like(q)
        rc = fn(q.data_ptr(), out.data_ptr(), kv.data_ptr(), kv.shape[0], bt.data_ptr(), bt.shape[1], cl.data_ptr(),
                q.shape[0], n_q, n_kv, 128 ** -0.5, pps, max_splits, 0, None,
                torch.cuda.current_stream().cuda_stream)
        assert rc == 0, lib.gllm_last_error().decode()
        ref = torch.zeros_like(q)
        ops.paged_decode(q, kv, bt, cl, n_q=n_q, n_kv=n_kv, out=ref, pages_per_split=pps)
        torch.cuda.synchronize()
        err = (out.float() - ref.float()).abs().max().item()
        assert err < 2e-2 * (ref.float().abs().max().item() + 1e-6), f"call {call}: max err {err}"
        oracle = ops.attention_ref(q, kv, bt, torch.arange(len(ctx), dtype=torch.int32, device=dev),
                                   (cl > 0).int(), cl, n_q, n_kv, 128 ** -0.5)
        assert (out.float() - oracle.float()).abs().max().item() < 2e-2 * (oracle.float().abs().max().item() + 1e-6)
        assert _status(lib) == 0, "the kernel recorded a problem on a well-formed call"


def test_noalloc_status_reports_a_bad_page_once():
    """A block-table entry outside the pool is redirected to page 0 and recorded in the path's status word; the read
    clears it, and the regular status word (the one the other tests' fixture checks) stays untouched."""
    from gllm_b200.ops import _native as nv
    dev = torch.device("cuda")
    lib, fn = _load()
    q, kv, bt, cl = _case(9, [40, 20], 8, 2, dev)
    bt[0, 1] = kv.shape[0] + 7          # outside the pool
    out = torch.zeros_like(q)
    rc = fn(q.data_ptr(), out.data_ptr(), kv.data_ptr(), kv.shape[0], bt.data_ptr(), bt.shape[1], cl.data_ptr(),
            q.shape[0], 8, 2, 128 ** -0.5, 4, 1, 0, None, torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    assert _status(lib) == 6            # ERR_BAD_PAGE
    assert _status(lib) == 0            # cleared by the read
    assert torch.isfinite(out.float()).all()
    assert nv.device_error() == 0


def test_noalloc_decode_rejects_oversize():
    dev = torch.device("cuda")
    lib, fn = _load()
    q, kv, bt, cl = _case(5, [16], 8, 2, dev)
    out = torch.zeros_like(q)
    # 4096 sequences x 8 heads x 8 splits is far beyond the built-in scratch: must fail cleanly, not launch
    rc = fn(q.data_ptr(), out.data_ptr(), kv.data_ptr(), kv.shape[0], bt.data_ptr(), bt.shape[1], cl.data_ptr(),
            4096, 8, 2, 128 ** -0.5, 4, 8, 0, None, torch.cuda.current_stream().cuda_stream)
    assert rc != 0
    assert b"exceeds the built-in" in lib.gllm_last_error()
