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


def test_fused_allreduce_world1_protocol():
    from gllm_b200.parallel.tensor_parallel import single_gpu_context
    dev = torch.device("cuda")
    H = 1024
    tp = single_gpu_context(dev, hidden=H, max_tokens=512)
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
        err = (x.float() - ref.float()).abs().max().item()
        assert err < 0.05 * ref.float().abs().max().item(), (it, err)
        torch.testing.assert_close(ss.sum(-1), x.float().pow(2).sum(-1), rtol=1e-3, atol=1e-3)
    assert int(tp._state[1]) == 5  # five launches advanced the launch state five times


@pytest.mark.multigpu
@pytest.mark.parametrize("mode", ["fused_p2p", "fused", "nccl", "fused_two_shot", "fused_p2p_two_shot"])
def test_fused_allreduce_two_gpus(mode):
    env = dict(os.environ, PYTHONPATH=ROOT, NCCL_NVLS_ENABLE=os.environ.get("NCCL_NVLS_ENABLE", "1"))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", str(29611 + hash(mode) % 200), os.path.join(ROOT, "tests", "tp_worker.py"), mode]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "TP_WORKER_OK" in r.stdout
