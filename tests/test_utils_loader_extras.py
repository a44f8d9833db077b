import json
import os

import torch

from gllm_b200.download import main as download_main
from gllm_b200.engine.batch import SequenceTelemetry
from gllm_b200.loader.static_compression import (prune_2_4, prune_dead_ffn_columns, pruning_error, sparsity_2_4_fraction)
from gllm_b200.loader.weight_tier import compress_tensor, decompress_tensor, plan_weight_tiers
from gllm_b200.utils import ChromeTrace, DeviceTimer, Flags, KernelRoofline, MetricsRegistry, Quantiles, apply_truncate_layers, nvtx_range
from gllm_b200.models.config import preset


def test_metrics_registry_and_roofline():
    q = Quantiles()
    for i in range(1, 101):
        q.add(float(i))
    s = q.summary()
    assert (s["p50"], s["p99"], s["max"], s["count"]) == (50.0, 99.0, 100.0, 100)
    m = MetricsRegistry()
    m.record_request(SequenceTelemetry(prompt_tokens=100, generated_tokens=20, cached_prefix_tokens=32, ttft_ms=12.0, tpot_ms=3.0, e2e_ms=70.0))
    m.record_request(SequenceTelemetry(prompt_tokens=60, generated_tokens=1, ttft_ms=8.0, e2e_ms=8.0))
    m.set("kv_pool_occupancy", 0.4)
    m.record_kernel("decode_attn", seconds=1e-3, bytes_moved=6.0e9)
    snap = json.loads(m.json_line(peak_gbs=6551.4, peak_tflops=1611.1))
    assert snap["counters"]["requests"] == 2 and snap["histograms"]["tpot_ms"]["count"] == 1
    assert abs(snap["prefix_hit_rate"] - 0.2) < 1e-9 and abs(snap["roofline"]["decode_attn"] - 0.9158) < 1e-3
    assert KernelRoofline("g", flops=1.6e12, seconds=2e-3).fraction(6551.4, 1600.0) == 0.5
    reg = m.export_prometheus()
    assert reg.get_sample_value("gllm_requests") == 2.0 and reg.get_sample_value("gllm_ttft_ms_p50") == 8.0


def test_tracing_and_flags(tmp_path, monkeypatch):
    with nvtx_range("noop"):
        pass
    t = DeviceTimer()
    with t.section("a"):
        sum(range(1000))
    assert t.results()["a"] >= 0 and t.max_over_ranks()["a"] == t.results()["a"]
    tr = ChromeTrace()
    with tr.span("step", tokens=5):
        pass
    tr.counter("kv", used=3)
    tr.save(str(tmp_path / "t.json"))
    ev = json.load(open(tmp_path / "t.json"))["traceEvents"]
    assert ev[0]["name"] == "step" and ev[0]["args"] == {"tokens": 5} and ev[1]["ph"] == "C"
    monkeypatch.setenv("GLLM_NAN_TRAP", "1"); monkeypatch.setenv("GLLM_TRUNCATE_LAYERS", "1")
    monkeypatch.setenv("GLLM_DUMP_LAYERS", "0,3"); monkeypatch.setenv("GLLM_CACHE_DIR", "/x/y")
    f = Flags.from_env()
    assert f.nan_trap and f.truncate_layers == 1 and f.dump_layers == [0, 3] and f.cache_dir == "/x/y" and not f.trace_swap
    assert apply_truncate_layers(preset("tiny-llama"), f).num_layers == 1


def test_weight_tiers_and_compression():
    sizes = {"L0.q_proj": 10, "L0.experts.0.up_proj": 40, "L0.experts.1.up_proj": 40, "L1.experts.0.up_proj": 40, "embed_tokens": 30}
    plan = {p.name: p.tier for p in plan_weight_tiers(sizes, device_budget=90, host_budget=40)}
    assert plan["embed_tokens"] == 1 and plan["L0.q_proj"] == 1 and sorted(plan.values()) == [1, 1, 1, 2, 3]
    t = torch.zeros(700, 1024, dtype=torch.bfloat16); t[::7] = 1.5
    pages, meta = compress_tensor(t)
    assert len(pages) == 2 and meta["compressed"] < meta["bytes"] // 10
    assert torch.equal(decompress_tensor(pages, meta), t)
    assert decompress_tensor(pages, meta, range(1, 2)).numel() == meta["bytes"] - (1 << 20)


def test_static_compression():
    torch.manual_seed(0)
    g, u, d = torch.randn(256, 32), torch.randn(256, 32), torch.randn(32, 256)
    g[10:100] = 0
    x = torch.randn(4, 32)
    want = (torch.nn.functional.silu(x @ g.t()) * (x @ u.t())) @ d.t()
    g2, u2, d2, rep = prune_dead_ffn_columns(g, u, d)
    assert rep.kept == 192 and rep.removed == 64 and g2.shape == (192, 32) and d2.shape == (32, 192)
    got = (torch.nn.functional.silu(x @ g2.t()) * (x @ u2.t())) @ d2.t()
    torch.testing.assert_close(got, want, rtol=1e-4, atol=1e-4)
    w = torch.randn(8, 64)
    p, mask = prune_2_4(w)
    assert mask.reshape(8, 16, 4).sum(-1).eq(2).all() and sparsity_2_4_fraction(p) == 1.0 and sparsity_2_4_fraction(w) == 0.0
    assert 0.1 < pruning_error(w, p) < 0.6


def test_download_cli_offline(tmp_path, capsys, monkeypatch):
    d = tmp_path / "org--model"
    d.mkdir()
    (d / "config.json").write_text("{}")
    assert download_main(["org/model", "--cache-dir", str(tmp_path)]) == 0
    assert str(d) in capsys.readouterr().out
    monkeypatch.setenv("HF_HUB_OFFLINE", "1")
    assert download_main(["org/absent", "--cache-dir", str(tmp_path)]) == 1


def test_static_compression_and_tier_plan_are_wired_into_loading():
    """``static_compression="dead_columns"`` drops dead FFN neurons when a layer is packed (same logits, narrower
    matrices), and a loaded model can plan its weight tiers for a device budget."""
    import torch
    from gllm_b200.engine.batch import ForwardBatch
    from gllm_b200.loader.loader import LoadedModel, WeightFormat
    from gllm_b200.models.config import preset
    from gllm_b200.models.decoder import DecoderModel
    from gllm_b200.models.weights import RandomWeights
    cfg = preset("tiny-qwen3")
    cfg.intermediate_size = 512
    src = RandomWeights(cfg, "cpu", torch.float32, seed=4, std=0.05)
    base_get = src.get

    def get(name):              # neurons 128..383 of every FFN are dead: zero gate rows
        t = base_get(name)
        if name.endswith("gate_proj"):
            t = t.clone()
            t[128:384] = 0
        return t
    src.get = get
    dense = DecoderModel(cfg, src, device="cpu", dtype=torch.float32, max_positions=64, weight_blob=False)
    cfg2 = preset("tiny-qwen3")
    cfg2.intermediate_size = 512
    cfg2.static_compression = "dead_columns"
    pruned = DecoderModel(cfg2, src, device="cpu", dtype=torch.float32, max_positions=64, weight_blob=False)
    assert dense.layers[0].w_down.shape[1] == 512 and pruned.layers[0].w_down.shape[1] == 256
    T = 7
    i32 = dict(dtype=torch.int32)
    fb = lambda: ForwardBatch(token_ids=torch.arange(T, **i32) + 5, positions=torch.arange(T, **i32),
                              slot_mapping=torch.arange(T, **i32), block_tables=torch.arange(2, **i32)[None],
                              ctx_lens=torch.tensor([T], **i32), q_start=torch.tensor([0], **i32),
                              q_len=torch.tensor([T], **i32), max_q_len=T)
    torch.testing.assert_close(pruned.forward(fb(), pruned.alloc_kv_cache(2)), dense.forward(fb(), dense.alloc_kv_cache(2)),
                               rtol=1e-4, atol=1e-4)

    class Shapes:
        shapes = {"embed_tokens": (1000, 64), "L0.q_proj": (64, 64), "L0.gate_proj": (4096, 64), "L1.gate_proj": (4096, 64)}
    lm = LoadedModel(path=None, format=WeightFormat.SAFETENSORS, config=cfg, weights=Shapes(), tokenizer=None)
    plan = {p.name: p.tier for p in lm.plan_tiers(device_budget=700_000, host_budget=600_000)}
    assert plan["embed_tokens"] == 1 and plan["L0.q_proj"] == 1          # always resident
    assert sorted([plan["L0.gate_proj"], plan["L1.gate_proj"]]) == [1, 2]   # one fits on the device, one goes to the host


def test_checkpoint_inspector_and_dump_comparison(tmp_path, capsys):
    import torch
    from gllm_b200.engine.guard import dump_tensors
    from gllm_b200.loader.gguf import write_gguf
    from gllm_b200.loader.describe import describe, main as inspect_main
    from gllm_b200.loader.safetensors import save_file
    from gllm_b200.utils.compare_dumps import compare, main as compare_main
    st = tmp_path / "m.safetensors"
    save_file({"model.embed_tokens.weight": torch.zeros(8, 4, dtype=torch.bfloat16), "model.norm.weight": torch.ones(4)}, st)
    d = describe(st)
    assert d["format"] == "safetensors" and len(d["tensors"]) == 2 and d["total_bytes"] == 8 * 4 * 2 + 4 * 4
    gg = tmp_path / "m.gguf"
    write_gguf(gg, {"general.architecture": "llama", "llama.block_count": 2}, {"token_embd.weight": torch.zeros(8, 32)})
    d = describe(gg)
    assert d["format"].startswith("gguf") and d["metadata"]["llama.block_count"] == 2 and d["tensors"][0]["shape"] == [8, 32]
    assert inspect_main([str(gg), "--tensors", "--keys", "--filter", "token"]) == 0
    assert "token_embd.weight" in capsys.readouterr().out
    a, b = tmp_path / "a", tmp_path / "b"
    x = torch.randn(4, 8)
    dump_tensors({"layer0/out": x, "layer1/out": x * 2}, str(a))
    dump_tensors({"layer0/out": x + 1e-5, "layer1/out": x * 2 + 0.5}, str(b))
    rows = compare(str(a), str(b))
    assert rows[0]["name"].startswith("layer1") and not rows[0]["ok"] and rows[1]["ok"]
    assert compare_main([str(a), str(b)]) == 1 and compare_main([str(a), str(a)]) == 0
