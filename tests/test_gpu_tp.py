"""Fused row-parallel GEMM + all-reduce kernel: single-GPU protocol test (world size 1 on ordinary device
memory: alternating buffers, arrival counter, launch state) and 2-GPU tests over NVLink (peer reds and
multimem), each against an fp32 reference. Run with -m gpu on a B200."""
import os
import subprocess
import sys

import pytest
import torch

from gllm_b200 import ops

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _rows_close(got, ref, what=""):
    """Per-row relative check: an error confined to a few rows or one tile column must not hide behind the maximum."""
    got, ref = got.float(), ref.float()
    row_err = (got - ref).abs().amax(-1)
    row_ref = ref.abs().amax(-1).clamp_min(1e-3)
    bad = (row_err > 0.03 * row_ref + 0.02).nonzero().flatten()
    assert bad.numel() == 0, f"{what}: rows {bad[:8].tolist()} off by {row_err[bad[:8]].tolist()}"


@pytest.mark.parametrize("mode", ["ll_p2p", "fused_p2p", "pull_p2p"])
def test_fused_allreduce_world1_protocol(mode):
    from gllm_b200.parallel.tensor_parallel import single_gpu_context
    dev = torch.device("cuda")
    H = 1024
    tp = single_gpu_context(dev, hidden=H, max_tokens=512, mode=mode)
    assert tp.mode == "fused" and not tp.uses_multimem
    torch.manual_seed(0)
    for it, (M, K) in enumerate([(256, 512), (100, 2048), (256, 512), (37, 1536), (512, 4096)]):
        a = torch.randn(M, K, device=dev).to(torch.bfloat16)
        w = (torch.randn(H, K, device=dev) * 0.05).to(torch.bfloat16)
        x = torch.randn(M, H, device=dev).to(torch.bfloat16)
        ref = (a.float() @ w.float().t() + x.float()).to(torch.bfloat16)
        ss_buf = torch.zeros(512, H // 256, device=dev)
        part = torch.empty(512, H, device=dev, dtype=torch.bfloat16)
        ss = tp.gemm_allreduce_residual(a, w, x, ss_buf, part, bn=256)
        _rows_close(x, ref, f"launch {it}")
        torch.testing.assert_close(ss.sum(-1), x.float().pow(2).sum(-1), rtol=1e-3, atol=1e-3)
    assert int(tp._state[1]) == 5  # five launches advanced the launch state five times


def test_low_latency_allreduce_prefill_sizes_world1():
    """The low-latency form with several tiles per CTA (M in the thousands: 256-wide tiles, rows stored by the epilogue
    warps tile after tile), interleaved with a decode-sized launch, world size 1 on ordinary memory."""
    from gllm_b200.parallel.tensor_parallel import single_gpu_context
    dev = torch.device("cuda")
    H = 1024
    tp = single_gpu_context(dev, hidden=H, max_tokens=4096, mode="ll_p2p")
    torch.manual_seed(6)
    for it, (M, K) in enumerate([(4096, 512), (3000, 1024), (256, 512), (4096, 512), (2049, 256)]):
        a = torch.randn(M, K, device=dev).to(torch.bfloat16)
        w = (torch.randn(H, K, device=dev) * 0.05).to(torch.bfloat16)
        x = torch.randn(M, H, device=dev).to(torch.bfloat16)
        ref = (a.float() @ w.float().t() + x.float()).to(torch.bfloat16)
        ss_buf = torch.zeros(4096, H // 256, device=dev)
        ss = tp.gemm_allreduce_residual(a, w, x, ss_buf, None)
        _rows_close(x, ref, f"launch {it} (M={M})")
        torch.testing.assert_close(ss.sum(-1), x.float().pow(2).sum(-1), rtol=1e-3, atol=1e-3)
    assert int(tp._state[1]) == 5


def test_push_allreduce_in_place_on_symmetric_buffers():
    """The serving path: x and the statistics live inside the symmetric region, nothing is staged."""
    from gllm_b200.parallel.tensor_parallel import single_gpu_context
    dev = torch.device("cuda")
    H = 2048
    tp = single_gpu_context(dev, hidden=H, max_tokens=1024)
    bufs = tp.workspace_buffers(1024)
    torch.manual_seed(1)
    for M, K in [(256, 1024), (1024, 512), (33, 2048)]:
        a = torch.randn(M, K, device=dev).to(torch.bfloat16)
        w = (torch.randn(H, K, device=dev) * 0.05).to(torch.bfloat16)
        x = bufs["x"][:M]
        x.copy_(torch.randn(M, H, device=dev).to(torch.bfloat16))
        ref = (a.float() @ w.float().t() + x.float()).to(torch.bfloat16)
        ss = tp.gemm_allreduce_residual(a, w, x, bufs["ss_a"][:M].reshape(-1)[:M * (H // 256)].view(M, H // 256), None)
        _rows_close(x, ref, f"M={M}")
        torch.testing.assert_close(ss.sum(-1), x.float().pow(2).sum(-1), rtol=1e-3, atol=1e-3)


@pytest.mark.parametrize("mode", ["ll_p2p", "fused_p2p"])
def test_push_allreduce_wait_runs_out_and_context_recovers(mode):
    """A wait on a flag (push form) or a data word (low-latency form) that nothing writes ends after the configured
    limit with a status code, the host sees it, and the next launch works (the permitted form of a failure test:
    nothing faults, traps or spins without a limit)."""
    from gllm_b200.ops import _native as nv
    from gllm_b200.parallel.tensor_parallel import single_gpu_context
    dev = torch.device("cuda")
    H, M, K = 1024, 64, 512
    tp = single_gpu_context(dev, hidden=H, max_tokens=256, mode=mode)
    torch.manual_seed(2)
    a = torch.randn(M, K, device=dev).to(torch.bfloat16)
    w = (torch.randn(H, K, device=dev) * 0.05).to(torch.bfloat16)
    x0 = torch.randn(M, H, device=dev).to(torch.bfloat16)
    ss_buf = torch.zeros(256, H // 256, device=dev)
    old = nv.set_wait_limits_ns(peer_ns=20_000_000)        # 20 ms
    nv.set_option("ar_drop_flags", 1)                      # the producers leave their tile flags unset
    try:
        x = x0.clone()
        t0 = torch.cuda.Event(enable_timing=True); t1 = torch.cuda.Event(enable_timing=True)
        t0.record()
        tp.gemm_allreduce_residual(a, w, x, ss_buf, None)
        t1.record()
        torch.cuda.synchronize()
        assert t0.elapsed_time(t1) < 2000.0                # it returned, and soon
        with pytest.raises(RuntimeError, match="timeout waiting for a peer"):
            nv.raise_on_device_error("after the dropped flags")
    finally:
        nv.set_option("ar_drop_flags", 0)
        nv.set_wait_limits_ns(*old)
    tp.reset()
    x = x0.clone()
    ref = (a.float() @ w.float().t() + x0.float()).to(torch.bfloat16)
    tp.gemm_allreduce_residual(a, w, x, ss_buf, None)
    torch.cuda.synchronize()
    _rows_close(x, ref, "after recovery")
    assert nv.device_error() == 0


def test_sequence_parallel_forms_world1_protocol():
    """All-gather in front of a GEMM and reduce-scatter behind one, world size 1 on ordinary memory: the slots, the
    parity sets and the launch counters of both forms over several launches, against fp32."""
    from gllm_b200.parallel.tensor_parallel import single_gpu_context
    dev = torch.device("cuda")
    H = 1024
    tp = single_gpu_context(dev, hidden=H, max_tokens=256, mode="ll_p2p")
    torch.manual_seed(4)
    for it, M in enumerate([256, 100, 256, 37]):
        x = torch.randn(M, H, device=dev).to(torch.bfloat16)
        w1 = (torch.randn(768, H, device=dev) * 0.05).to(torch.bfloat16)
        w2 = (torch.randn(H, 768, device=dev) * 0.05).to(torch.bfloat16)
        a_full = torch.zeros(M, H, device=dev, dtype=torch.bfloat16)
        tp.allgather_input(x, a_full)
        mid = ops.gemm(a_full, w1, bn=128)
        assert torch.equal(a_full, x), f"launch {it}: gathered rows differ"
        _rows_close(mid, x.float() @ w1.float().t(), f"all-gather GEMM, launch {it}")
        res = x.clone()
        ss = torch.zeros(M, H // 256, device=dev)
        tp.gemm_reduce_scatter_residual(mid, w2, res, ss, M)
        _rows_close(res, mid.float() @ w2.float().t() + x.float(), f"reduce-scatter GEMM, launch {it}")
        torch.testing.assert_close(ss.sum(-1), res.float().pow(2).sum(-1), rtol=2e-3, atol=2e-3)
    assert int(tp._ag_state[0]) == 4 and int(tp._state[1]) == 4


@pytest.mark.parametrize("fmt", ["mxfp8", "nvfp4"])
def test_blockscaled_gemm_with_fused_allreduce_world1(fmt):
    """The block-scaled row-parallel GEMM with the low-latency all-reduce in its epilogue, one rank: parked tiles at
    decode sizes, staged rows at prefill sizes, per-tensor scales of NVFP4 carried by the partials; against the
    block-scaled residual GEMM without the all-reduce and against fp32 on the dequantised operands."""
    from gllm_b200.ops import _native as nv
    from gllm_b200.ops import blockscale as B
    from gllm_b200.parallel.tensor_parallel import single_gpu_context
    dev = torch.device("cuda")
    H, K = 2048, 1024
    tp = single_gpu_context(dev, hidden=H, max_tokens=2048, mode="ll_p2p")
    torch.manual_seed(8)
    w = B.quantize((torch.randn(H, K) * 0.05).to(torch.bfloat16), fmt).to(dev)
    for it, M in enumerate([256, 77, 1500, 256]):
        a = torch.randn(M, K, device=dev).to(torch.bfloat16)
        aq = B.quantize_act(a, fmt, tensor_scale=1.0 / 64.0) if fmt == "nvfp4" else B.quantize_act(a, fmt)
        x0 = torch.randn(M, H, device=dev).to(torch.bfloat16)
        assert tp.can_fuse_blockscaled(M, H)
        x = x0.clone()
        ss = tp.gemm_allreduce_residual_bs(aq, w, x, torch.zeros(M, H // 128, device=dev))
        want, _ = B.gemm_residual(aq, w, x0)
        torch.cuda.synchronize()
        _rows_close(x, want.float(), f"{fmt} launch {it} (M={M}) against the plain residual GEMM")
        ref = aq.dequantize()[:M].float() @ w.dequantize().float().t() + x0.float()
        _rows_close(x, ref, f"{fmt} launch {it} (M={M}) against fp32")
        torch.testing.assert_close(ss.sum(-1), x.float().pow(2).sum(-1), rtol=2e-3, atol=2e-3)
    assert nv.device_error() == 0


def test_allgather_statistics_feed_the_gemm_of_the_same_launch():
    """The all-gather phase writes the gathered rows' sums of squares per 256 columns; the GEMM behind it (same launch)
    normalises its rows with them: QKV and GLU epilogues against the fp32 product of the normalised rows."""
    from gllm_b200.ops import _native as nv
    from gllm_b200.parallel.tensor_parallel import single_gpu_context
    dev = torch.device("cuda")
    H = 1024
    tp = single_gpu_context(dev, hidden=H, max_tokens=256, mode="ll_p2p")
    torch.manual_seed(6)
    for it, M in enumerate([256, 77, 129]):
        x = torch.randn(M, H, device=dev).to(torch.bfloat16)
        w1 = (torch.randn(768, H, device=dev) * 0.05).to(torch.bfloat16)
        a_full = torch.zeros(M, H, device=dev, dtype=torch.bfloat16)
        ss = torch.zeros(M, H // 256, device=dev)
        tp.allgather_input(x, a_full, ss_out=ss)
        mid = ops.gemm(a_full, w1, bn=128, row_ss=ss, norm_dim=H, eps=1e-6)
        torch.cuda.synchronize()
        assert torch.equal(a_full, x)
        torch.testing.assert_close(ss.sum(-1), x.float().pow(2).sum(-1), rtol=1e-4, atol=1e-3)
        xn = x.float() * torch.rsqrt(x.float().pow(2).mean(-1, keepdim=True) + 1e-6)
        _rows_close(mid, xn @ w1.float().t(), f"normalised all-gather GEMM, launch {it}")
    assert nv.device_error() == 0


def test_sequence_parallel_decoder_world1_matches_plain_model():
    """The sequence-parallel layer (gather + QKV, o_proj + scatter, gather + gate/up, down + scatter as four fused
    kernels) with one rank against the ordinary fused layer: same logits, same cache."""
    from gllm_b200.engine.batch import ForwardBatch
    from gllm_b200.models.config import preset
    from gllm_b200.models.decoder import DecoderModel
    from gllm_b200.models.weights import RandomWeights
    from gllm_b200.ops import _native as nv
    from gllm_b200.parallel.tensor_parallel import single_gpu_context
    dev = torch.device("cuda")
    cfg = preset("tiny-qwen3")
    cfg.hidden_size, cfg.num_heads, cfg.num_kv_heads, cfg.head_dim = 1024, 8, 2, 128
    cfg.intermediate_size, cfg.num_layers, cfg.vocab_size = 2048, 3, 2048
    src = RandomWeights(cfg, "cpu", torch.float32, seed=5, std=0.04)
    tp = single_gpu_context(dev, hidden=cfg.hidden_size, max_tokens=256, mode="ll_p2p")
    sp = DecoderModel(cfg, src, device=dev, dtype=torch.bfloat16, tp=tp, max_positions=512, sequence_parallel=True)
    plain = DecoderModel(cfg, src, device=dev, dtype=torch.bfloat16, max_positions=512)

    def i32(v):
        return torch.as_tensor(v, dtype=torch.int32, device=dev)
    for T in (256, 77, 1):
        ids = ((torch.arange(T, dtype=torch.int32) * 7 + 3) % cfg.vocab_size).to(dev)
        def batch():
            return ForwardBatch(token_ids=ids, positions=i32(list(range(T))), slot_mapping=i32(list(range(T))),
                                block_tables=i32([list(range(16))]), ctx_lens=i32([T]), q_start=i32([0]),
                                q_len=i32([T]), max_q_len=T)
        kv_a, kv_b = sp.alloc_kv_cache(16), plain.alloc_kv_cache(16)
        got = sp.forward(batch(), kv_a).float()
        want = plain.forward(batch(), kv_b).float()
        torch.cuda.synchronize()
        _rows_close(got, want, f"sequence-parallel logits, T={T}")
        for a, b in zip(kv_a, kv_b):
            torch.testing.assert_close(a.float(), b.float(), rtol=0.05, atol=0.05)
    assert nv.device_error() == 0


@pytest.mark.multigpu
def test_context_parallel_prefill_two_gpus():
    """Two ranks prefill halves of the prompts (tcgen05 attention over the exchanged pages) against one rank."""
    env = dict(os.environ, PYTHONPATH=ROOT, NCCL_NVLS_ENABLE=os.environ.get("NCCL_NVLS_ENABLE", "1"))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", "29885", os.path.join(ROOT, "tests", "cp_worker.py"), "cuda"]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert r.stdout.count("CP_WORKER_OK") == 2


@pytest.mark.multigpu
@pytest.mark.parametrize("fmt", ["mxfp8", "nvfp4"])
def test_blockscaled_gemm_with_fused_allreduce_two_gpus(fmt):
    env = dict(os.environ, PYTHONPATH=ROOT, NCCL_NVLS_ENABLE=os.environ.get("NCCL_NVLS_ENABLE", "1"))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", str(29881 + (fmt == "nvfp4")), os.path.join(ROOT, "tests", "tp_bs_worker.py"),
           "ll", fmt]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "TP_BS_WORKER_OK" in r.stdout


@pytest.mark.multigpu
@pytest.mark.parametrize("mode", ["ll", "nccl"])
def test_sequence_parallel_decoder_two_gpus(mode):
    env = dict(os.environ, PYTHONPATH=ROOT, NCCL_NVLS_ENABLE=os.environ.get("NCCL_NVLS_ENABLE", "1"))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", str(29871 + (mode == "ll")), os.path.join(ROOT, "tests", "sp_decoder_worker.py"),
           mode]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert r.stdout.count("SP_DECODER_WORKER_OK") == 2


@pytest.mark.multigpu
@pytest.mark.parametrize("mode", ["ll", "ll_p2p", "nccl"])
def test_sequence_parallel_block_two_gpus(mode):
    env = dict(os.environ, PYTHONPATH=ROOT, NCCL_NVLS_ENABLE=os.environ.get("NCCL_NVLS_ENABLE", "1"))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", str(29911 + hash(mode) % 50), os.path.join(ROOT, "tests", "sp_worker.py"), mode]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert r.stdout.count("SP_WORKER_OK") == 2


@pytest.mark.multigpu
@pytest.mark.parametrize("mode", ["ll", "fused_p2p", "fused", "nccl", "pull", "pull_p2p", "pull_two_shot", "pull_p2p_two_shot"])
def test_fused_allreduce_two_gpus(mode):
    env = dict(os.environ, PYTHONPATH=ROOT, NCCL_NVLS_ENABLE=os.environ.get("NCCL_NVLS_ENABLE", "1"))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", str(29611 + hash(mode) % 200), os.path.join(ROOT, "tests", "tp_worker.py"), mode]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "TP_WORKER_OK" in r.stdout
