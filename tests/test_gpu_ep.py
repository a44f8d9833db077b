"""Expert-parallel dispatch/combine kernels: world size 1 on ordinary device memory (the protocol: counts,
row plan, peer stores, return scatter, flag epochs) and 2-GPU runs over NVLink, fused and all-to-all, each
against the fp32 CPU oracle of the full MoE layer. Run with -m gpu on a B200."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(world, mode, port):
    env = dict(os.environ, PYTHONPATH=ROOT)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr",
           "127.0.0.1", "--master-port", str(port), os.path.join(ROOT, "tests", "ep_worker.py"), mode]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert r.stdout.count("EP_WORKER_OK") == world, r.stdout[-2000:]


def test_ep_fused_world1_protocol():
    _run(1, "fused", 29831)


@pytest.mark.multigpu
@pytest.mark.parametrize("mode", ["fused", "a2a"])
def test_ep_two_gpus(mode):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    _run(2, mode, 29832 + (mode == "a2a"))


@pytest.mark.multigpu
def test_tp_attention_plus_expert_sharded_moe_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    env = dict(os.environ, PYTHONPATH=ROOT)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29839", os.path.join(ROOT, "tests", "tp_moe_worker.py"), "gpu"]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=400)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert r.stdout.count("TP_MOE_WORKER_OK") == 2


@pytest.mark.multigpu
def test_lockstep_engines_with_fused_expert_parallel_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    env = dict(os.environ, PYTHONPATH=ROOT)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29841", os.path.join(ROOT, "tests", "ep_engine_worker.py"), "gpu"]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=400)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert r.stdout.count("EP_ENGINE_WORKER_OK") == 2
