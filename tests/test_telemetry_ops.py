import pytest
import torch

from gllm_b200.ops.telemetry import layer_telemetry, requant_pages_


def _case(dev, dtype):
    torch.manual_seed(0)
    x = torch.randn(64, 128).to(dtype).to(dev)
    y = (x.float() * 1.05).to(dtype)
    act = torch.randn(64, 256).to(dtype).to(dev)
    act[:, :64] = 0
    return x, y, act


def test_layer_telemetry_and_requant_cpu():
    x, y, act = _case("cpu", torch.float32)
    t = layer_telemetry(x, y, act)
    assert abs(t["delta_rho"] - 0.05) < 1e-4 and abs(t["sparsity"] - 0.25) < 0.01
    cache = torch.randn(6, 2, 2, 16, 32)
    before = cache.clone()
    requant_pages_(cache, [1, 4], "kivi4")
    assert torch.equal(cache[0], before[0]) and not torch.equal(cache[1], before[1])
    assert (cache[1] - before[1]).abs().max() < (before[1].amax() - before[1].amin()) / 15
    requant_pages_(cache, [2], "fp8")
    assert (cache[2] - before[2]).abs().max() < 0.07 * before[2].abs().max()
    levels = cache[4].reshape(-1, 32)[0].unique().numel()
    assert levels <= 16


@pytest.mark.gpu
def test_layer_telemetry_and_requant_gpu_match_cpu():
    x, y, act = _case("cuda", torch.bfloat16)
    g = layer_telemetry(x, y, act)
    c = layer_telemetry(x.cpu(), y.cpu(), act.cpu())
    assert abs(g["delta_rho"] - c["delta_rho"]) < 1e-3 and abs(g["sparsity"] - c["sparsity"]) < 1e-4
    cache = torch.randn(6, 2, 2, 16, 32).to(torch.bfloat16)
    for tier in ("fp8", "kivi4", "kivi2"):
        a = requant_pages_(cache.clone().cuda(), [1, 4], tier).float().cpu()
        b = requant_pages_(cache.clone(), [1, 4], tier).float()
        assert torch.equal(a[0], b[0])
        assert (a - b).abs().max() <= (0.02 if tier == "fp8" else 0.51) * (cache.float().amax() - cache.float().amin()) / (15 if tier != "kivi2" else 3) + 0.02
    from gllm_b200.ops import _native as nv
    assert nv.device_error() == 0
