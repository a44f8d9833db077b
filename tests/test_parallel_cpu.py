"""Distributed logic as pure functions of (rank, world) plus gloo multi-process checks on CPU."""
import os
import subprocess
import sys
import textwrap

import pytest
import torch

from gllm_b200.parallel import config as C
from gllm_b200.parallel import pipeline as P
from gllm_b200.parallel.comm import CommError, CommHandle
from gllm_b200.parallel.context_parallel import CpConfig, RingAttention, merge_partials, partial_attention, ring_steps, shard_bounds
from gllm_b200.parallel.pd import kv_dist_plan, resolve_pd_role
from gllm_b200.models.weights import shard_kind, shard_range, shard_tensor
from gllm_b200.moe.eplb import Eplb, dispatch_experts, make_placement
from gllm_b200.moe.routing import (ExpertLoadBalancer, ExpertRouteConfig, ExpertRouteTable, ExpertThermalTracker,
                                   MoeHardwareDispatcher, load_balance_loss)

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_parallel_config_validation_and_topology():
    with pytest.raises(C.ConfigError):
        C.ParallelConfig(tp=4, pp=2).validate(6)
    with pytest.raises(C.ConfigError):
        C.ParallelConfig(tp=4, pp=2, ep=3).validate(8)
    cfg = C.ParallelConfig(tp=4, pp=2, ep=4)
    topo = C.Topology(cfg, 8)
    assert topo.coord(5) == C.RankCoord(5, tp=1, cp=0, pp=1, ep=1)
    assert topo.tp_group(5) == [4, 5, 6, 7] and topo.pp_group(5) == [1, 5] and topo.ep_group(6) == [4, 5, 6, 7]
    assert topo.pp_next(1) == 5 and topo.pp_next(5) is None and topo.pp_prev(5) == 1 and topo.is_tp_master(4)
    assert topo.all_groups("tp") == [[0, 1, 2, 3], [4, 5, 6, 7]] and len(topo.all_groups("pp")) == 4
    t3 = C.Topology(C.ParallelConfig(tp=2, cp=2, pp=2, ep=2), 8)
    assert t3.cp_group(1) == [1, 3] and t3.tp_group(6) == [6, 7] and t3.coord(7).pp == 1
    assert C.select_algorithm(1 << 20, 8, True, False) == C.CommAlgorithm.HARDWARE_REDUCE
    assert C.select_algorithm(1 << 20, 8, True, True) == C.CommAlgorithm.FLUX_PIPELINE
    assert C.select_algorithm(4096, 8, False, False) == C.CommAlgorithm.DIRECT
    C.DistributedConfig(parallel=C.ParallelConfig(tp=8)).validate(8)


def test_comm_handle_without_backend_errors():
    h = CommHandle.new_for_test(3, 8)
    assert (h.rank, h.world_size) == (3, 8)
    for fn in (lambda: h.all_reduce(torch.zeros(1)), lambda: h.barrier(), lambda: h.send(torch.zeros(1), 0),
               lambda: h.all_gather(torch.zeros(8), torch.zeros(1))):
        with pytest.raises(CommError):
            fn()
    h.destroy()  # idempotent on an uninitialised handle


def test_tp_shard_rules():
    assert shard_kind("L3.q_proj") == "column" and shard_kind("L3.down_proj") == "row" and shard_kind("L3.input_norm") == "replicated"
    assert shard_kind("L0.router") == "replicated" and shard_kind("lm_head") == "column" and shard_kind("L1.kv_b_proj") == "column"
    assert [shard_range(10, r, 4) for r in range(4)] == [(0, 3), (3, 6), (6, 8), (8, 10)]
    w = torch.arange(8 * 6, dtype=torch.float32).reshape(8, 6)
    parts = [shard_tensor("L0.q_proj", w, r, 2, head_dim=2) for r in range(2)]
    assert torch.equal(torch.cat(parts, 0), w) and parts[0].shape == (4, 6)
    rows = [shard_tensor("L0.o_proj", w, r, 3, head_dim=2) for r in range(3)]
    assert torch.equal(torch.cat(rows, 1), w) and rows[1].shape == (8, 2)
    assert shard_tensor("L0.input_norm", w, 1, 2) is w
    # row-parallel sum of partial products equals the full product
    x = torch.randn(5, 6)
    full = x @ w.t()
    acc = sum(x[:, r * 2:(r + 1) * 2] @ rows[r].t() for r in range(3))
    torch.testing.assert_close(acc, full)


def test_pipeline_config_schedules_and_bubbles():
    pc = P.PipelineConfig(num_layers=10, num_stages=4)
    assert [list(r) for r in pc.stage_ranges()] == [[0, 1, 2], [3, 4, 5], [6, 7], [8, 9]]
    assert pc.stage_of_layer(7) == 2
    il = P.PipelineConfig(num_layers=8, num_stages=2, virtual_stages=2)
    assert [list(r) for r in il.layers_of_stage(1)] == [[2, 3], [6, 7]]
    costs = P.PipelineConfig(num_layers=4, num_stages=2, layer_costs=[4, 1, 1, 1]).stage_ranges()
    assert [list(r) for r in costs] == [[0], [1, 2, 3]]
    assert P.pp_weight_filter("L3.q_proj", range(2, 5), False, False) and not P.pp_weight_filter("L7.q_proj", range(2, 5), False, False)
    assert P.pp_weight_filter("embed_tokens", range(0, 2), True, False) and not P.pp_weight_filter("lm_head", range(0, 2), True, False)
    assert P.pp_weight_filter("embed_tokens", range(6, 8), False, True, tied=True)
    assert P.split_micro_batches(10, 4) == [(0, 3), (3, 3), (6, 2), (8, 2)]
    g = P.gpipe_schedule(0, 4, 6)
    assert [o.micro for o in g] == list(range(6)) and [o.phase for o in g][:3] == ["warmup"] * 3
    f1b = P.one_f_one_b_schedule(1, 4, 6)
    kinds = "".join(o.kind.value for o in f1b)
    assert kinds.startswith("FF") and kinds.count("F") == 6 and kinds.count("B") == 6 and "FBFB" in kinds
    assert [o.micro for o in f1b if o.kind == P.OpKind.BACKWARD] == list(range(6))
    assert all(o.kind == P.OpKind.FORWARD for o in P.one_f_one_b_schedule(1, 4, 6, forward_only=True))
    iv = P.interleaved_schedule(0, 2, 4, 2)
    assert len(iv) == 8 and {(o.micro, o.chunk) for o in iv} == {(m, c) for m in range(4) for c in range(2)}
    zb = P.zero_bubble_schedule(3, 4, 4)
    assert sum(o.kind == P.OpKind.BACKWARD_WEIGHT for o in zb) == 4
    assert abs(P.bubble_fraction(4, 12) - 3 / 15) < 1e-9 and P.bubble_fraction(4, 12, 2) < P.bubble_fraction(4, 12)
    assert P.choose_micro_batches(8192, 2, 0.05) >= 19 or P.choose_micro_batches(8192, 2, 0.05) * 256 <= 8192
    m = P.overlap_model(10.0, 4.0, "auto", 0.3)
    assert m["exposed_comm_ms"] == 0.0 and m["step_ms"] > 10.0
    assert P.overlap_model(10.0, 4.0, "serial")["step_ms"] == 14.0
    kvm = P.StageKvManager(0, range(0, 4), 1024, 1024 * 4 * 100)
    assert kvm.capacity_tokens() == 100 and kvm.reserve(60) and not kvm.reserve(50) and kvm.reserve(40)


def test_stage_fault_recovery_with_fake_clock():
    fr = P.StageFaultRecovery(4, P.HeartbeatConfig(interval_s=1, timeout_s=3, max_consecutive_misses=3))
    for s in range(4):
        fr.heartbeat(s, now=100.0)
    for s in (0, 1, 3):
        fr.heartbeat(s, now=104.0)
    st = fr.detect(now=104.5)
    assert st[2] == P.StageStatus.FAULTED and st[0] == P.StageStatus.HEALTHY
    fr.isolate(2)
    fr.heartbeat(2, now=105.0)                      # an isolated stage cannot vote itself back in
    assert fr.status[2] == P.StageStatus.ISOLATED
    pc = P.PipelineConfig(num_layers=8, num_stages=4)
    plan = fr.plan_migration(2, pc, bytes_per_layer=10 ** 9, kv_bytes=5 * 10 ** 8)
    assert plan.layers == [4, 5] and plan.target_stage in (1, 3) and plan.estimated_s > 0
    before = {s: list(r) for s, r in enumerate(pc.stage_ranges())}
    after = {0: [0, 1], 1: [2, 3, 4, 5], 3: [6, 7]}
    assert P.StageFaultRecovery.verify_post_migration_equivalence(before, after)
    assert not P.StageFaultRecovery.verify_post_migration_equivalence(before, {0: [0, 1], 1: [2, 3], 3: [6, 7]})


def test_ring_attention_plan_and_single_process_equivalence():
    assert [shard_bounds(10, 4, r) for r in range(4)] == [(0, 3), (3, 6), (6, 8), (8, 10)]
    assert ring_steps(CpConfig(4, 0), 64) == [0] and ring_steps(CpConfig(4, 3), 64) == [3, 2, 1, 0]
    assert ring_steps(CpConfig(4, 3, sliding_window=16), 64) == [3, 2]      # older blocks fall outside the window
    assert ring_steps(CpConfig(4, 1), 64, causal=False) == [1, 0, 3, 2]
    torch.manual_seed(0)
    T, H, Hkv, D = 37, 4, 2, 16
    q, k, v = torch.randn(T, H, D), torch.randn(T, Hkv, D), torch.randn(T, Hkv, D)
    pos = torch.arange(T)
    full, _ = partial_attention(q, k, v, pos, pos, D ** -0.5)
    # emulate the ring in one process: merge the partials of each KV shard
    for cp in (2, 3):
        outs = []
        for r in range(cp):
            a, b = shard_bounds(T, cp, r)
            o = torch.zeros(b - a, H, D); lse = torch.full((b - a, H), float("-inf"))
            for src in ring_steps(CpConfig(cp, r), T):
                c, d = shard_bounds(T, cp, src)
                po, pl = partial_attention(q[a:b], k[c:d], v[c:d], pos[a:b], pos[c:d], D ** -0.5)
                o, lse = merge_partials(o, lse, po, pl)
            outs.append(o)
        torch.testing.assert_close(torch.cat(outs), full, rtol=1e-4, atol=1e-5)


def test_pd_roles_and_kv_dist_modes():
    assert resolve_pd_role(C.PdRole.PREFILL_ONLY, True, True) == {"prefill": True, "decode": False, "ship_kv": True}
    assert resolve_pd_role(C.PdRole.DECODE_ONLY, True, True)["prefill"] is False
    assert resolve_pd_role(C.PdRole.COLLOCATED, True, False) == {"prefill": True, "decode": False, "ship_kv": False}
    assert kv_dist_plan(C.KvDistMode.MIRROR, 1, 4, 8)["mirror_to"] == [0, 2, 3]
    assert kv_dist_plan(C.KvDistMode.PARTIAL_HEAD_MIRROR, 2, 4, 8)["store_heads"] == [4, 5]
    assert kv_dist_plan(C.KvDistMode.TIERED_CACHE, 0, 2, 8).get("tiered")


def test_expert_placement_dispatch_eplb_and_routing_tables():
    mc = C.MoeDistConfig(placement=C.MoePlacement.ROUND_ROBIN)
    assert make_placement(mc, 8, 4).owner == [0, 1, 2, 3, 0, 1, 2, 3]
    auto = make_placement(C.MoeDistConfig(), 8, 4)
    assert auto.owner == [0, 0, 1, 1, 2, 2, 3, 3] and auto.local_experts(2) == [4, 5]
    hc = make_placement(C.MoeDistConfig(placement=C.MoePlacement.HOT_COLD, hot_experts=[5]), 8, 4)
    assert hc.ranks_of(5) == [2, 0, 1, 3] and 5 in hc.local_experts(0)
    ids = torch.tensor([[0, 5], [7, 5], [2, 3]])
    by_rank = dispatch_experts(ids, hc, rank=0, world=4)
    assert by_rank[0] == [0, 1, 3] and by_rank[3] == [2] and by_rank[1] == [4, 5]      # hot expert 5 stays local
    clock = [0.0]
    eplb = Eplb(8, window_s=60, threshold=2.0, clock=lambda: clock[0])
    eplb.record(torch.tensor([100, 1, 1, 1, 1, 1, 1, 1]))
    clock[0] = 30.0
    eplb.record(torch.tensor([100, 1, 1, 1, 1, 1, 1, 1]))
    tot = eplb.aggregate()
    assert eplb.imbalance(tot) > 2.0
    new = eplb.decide(tot, C.MoeDistConfig())
    assert new.placement == C.MoePlacement.HOT_COLD and new.hot_experts == [0]
    clock[0] = 200.0
    eplb.record(torch.ones(8, dtype=torch.int64))
    assert eplb.decide(eplb.aggregate(), C.MoeDistConfig()) is None     # old samples aged out of the window
    rc = ExpertRouteConfig(num_experts=4, top_k=2, capacity_factor=1.0)
    assert rc.expert_capacity(8) == 4
    lg = torch.zeros(8, 4); lg[:, 0] = 5.0; lg[:, 1] = 4.0
    tab = ExpertRouteTable.from_gate_logits(rc, lg, enforce_capacity=True)
    assert tab.counts()[0] == 4 and sum(len(r.dropped) for r in tab.routes) == 8
    assert len(tab.tokens_for_expert(0)) == 4
    assert load_balance_loss(torch.zeros(64, 4), 2) == pytest.approx(1.0, rel=1e-3) and load_balance_loss(lg, 2) > 1.5
    lb = ExpertLoadBalancer(4, window=4)
    lb.record([10, 1, 1, 0]); lb.record([12, 0, 1, 0])
    assert lb.hot_experts() == [0] and lb.cold_experts() == [3] and abs(sum(lb.hit_rates()) - 1) < 1e-9
    plan = MoeHardwareDispatcher([0, 1], max_cpu_ratio=0.5, cpu_enabled=True).dispatch([10, 5, 3, 9])
    assert [a.expert_idx for a in plan.gpu_experts] == [0, 1] and [a.expert_idx for a in plan.cpu_experts] == [3, 2]
    th = ExpertThermalTracker(3)
    for _ in range(5):
        th.step([3, 0, 0])
    assert th.state(0) == "hot" and th.state(1) == "cold" and th.eviction_candidates(1) in ([1], [2])


WORKER = textwrap.dedent('''
    import os, sys, torch, torch.distributed as dist
    sys.path.insert(0, os.environ["GLLM_ROOT"])
    from gllm_b200.parallel.comm import CommHandle
    from gllm_b200.parallel.context_parallel import CpConfig, RingAttention, partial_attention, shard_bounds
    from gllm_b200.parallel.pipeline import ActivationTransport
    from gllm_b200.parallel.pd import KvPageTransport, SaguaroLink
    h = CommHandle.from_env("gloo", timeout_s=60)
    r, w = h.rank, h.world_size
    t = torch.full((4,), float(r + 1)); h.all_reduce(t); assert t[0] == w * (w + 1) / 2
    c = h.all_reduce_counts(torch.tensor([r, 1])); assert c.tolist() == [w * (w - 1) // 2, w]
    out = torch.empty(w * 2); h.all_gather(out, torch.full((2,), float(r))); assert out.tolist() == [float(i // 2) for i in range(2 * w)]
    rs = torch.empty(2); h.reduce_scatter(rs, torch.arange(2 * w, dtype=torch.float32)); assert rs.tolist() == [w * (2 * r), w * (2 * r + 1)]
    # ring attention across ranks == single-process attention
    torch.manual_seed(0)
    T, H, Hkv, D = 41, 4, 2, 16
    q, k, v = torch.randn(T, H, D), torch.randn(T, Hkv, D), torch.randn(T, Hkv, D)
    a, b = shard_bounds(T, w, r)
    o = RingAttention(CpConfig(w, r), h).run(q[a:b], k[a:b], v[a:b], T)
    pos = torch.arange(T)
    full, _ = partial_attention(q, k, v, pos, pos, D ** -0.5)
    assert (o - full[a:b]).abs().max() < 1e-4, (o - full[a:b]).abs().max()
    # pipeline activations (int8 on the wire) and KV pages between neighbours; SAGUARO hand-off
    if w >= 2 and r < 2:
        tr = ActivationTransport(h, prev_rank=0 if r == 1 else None, next_rank=1 if r == 0 else None, hidden=8, device="cpu",
                                 dtype=torch.float32, quant="int8", max_tokens=16)
        x = torch.arange(40, dtype=torch.float32).reshape(5, 8)
        if r == 0:
            for wk in tr.send(x): wk.wait()
        else:
            y = tr.recv(5); assert (y - x).abs().max() <= x.abs().max() / 127 + 1e-6
        kv = [torch.full((6, 2, 1, 16, 4), float(r * 10 + l)) for l in range(2)]
        kt = KvPageTransport(h, kv)
        if r == 0: kt.send_pages([1, 4], 1)
        else:
            res = kt.recv_pages([0, 5], 0); assert res.pages == 2 and kv[1][5, 0, 0, 0, 0] == 1.0 and kv[0][1, 0, 0, 0, 0] == 10.0
        link = SaguaroLink(h, draft_rank=0, verify_rank=1)
        if r == 0:
            link.send_draft([5, 6, 7]); assert link.recv_verdict() == (2, 9)
        else:
            assert link.recv_draft() == [5, 6, 7]; link.send_verdict(2, 9)
    h.barrier()
    print("WORKER_OK", r, flush=True)
    h.destroy()
''')


@pytest.mark.parametrize("world", [2, 3])
def test_gloo_collectives_ring_attention_and_transports(tmp_path, world):
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    env = dict(os.environ, GLLM_ROOT=ROOT, MASTER_ADDR="127.0.0.1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr",
           "127.0.0.1", "--master-port", str(29700 + world), str(script)]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=240)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    assert r.stdout.count("WORKER_OK") == world


def test_rank_failure_is_detected_on_the_host(tmp_path):
    """A rank that exits before a collective: the survivor's collective ends with an error within the timeout
    (no GPU involved, gloo)."""
    script = tmp_path / "fail.py"
    script.write_text(textwrap.dedent('''
        import os, sys, time, torch, torch.distributed as dist
        sys.path.insert(0, os.environ["GLLM_ROOT"])
        from gllm_b200.parallel.comm import CommHandle
        h = CommHandle.from_env("gloo", timeout_s=5)
        h.barrier()
        if h.rank == 1:
            os._exit(0)            # leaves between steps, nothing in flight
        t0 = time.time()
        try:
            h.all_reduce(torch.ones(1))
            print("NO_ERROR")
        except Exception as e:
            print("SURVIVOR_SAW_ERROR", round(time.time() - t0, 1), flush=True)
        os._exit(0)
    '''))
    env = dict(os.environ, GLLM_ROOT=ROOT, MASTER_ADDR="127.0.0.1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29741", str(script)]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=120)
    assert "SURVIVOR_SAW_ERROR" in r.stdout, r.stdout[-1500:] + r.stderr[-1500:]


@pytest.mark.parametrize("world", [2, 4])
def test_expert_parallel_all_to_all_matches_full_layer(world):
    """Every rank routes its own tokens; experts are split over the ranks; result equals the unsplit layer."""
    env = dict(os.environ, PYTHONPATH=ROOT, MASTER_ADDR="127.0.0.1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr",
           "127.0.0.1", "--master-port", str(29760 + world), os.path.join(ROOT, "tests", "ep_worker.py"), "cpu"]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    assert r.stdout.count("EP_WORKER_OK") == world


@pytest.mark.parametrize("world", [2, 4])
def test_pipeline_parallel_generation_matches_single_process(world):
    env = dict(os.environ, PYTHONPATH=ROOT, MASTER_ADDR="127.0.0.1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr",
           "127.0.0.1", "--master-port", str(29780 + world), os.path.join(ROOT, "tests", "pp_worker.py"), "cpu"]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=400)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    assert r.stdout.count("PP_WORKER_OK") == world


@pytest.mark.parametrize("world", [2])
def test_serving_engine_as_pipeline_stages_matches_single_process(world):
    """The real LLMEngine (C++ batcher, paged KV, chunked prefill) run as pipeline stages over gloo."""
    env = dict(os.environ, PYTHONPATH=ROOT, MASTER_ADDR="127.0.0.1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr",
           "127.0.0.1", "--master-port", str(29820 + world), os.path.join(ROOT, "tests", "pp_engine_worker.py"), "cpu"]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=400)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    assert r.stdout.count("PP_ENGINE_WORKER_OK") == world


def test_tp_attention_with_expert_sharded_moe_matches_unsplit_model():
    env = dict(os.environ, PYTHONPATH=ROOT, MASTER_ADDR="127.0.0.1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29795", os.path.join(ROOT, "tests", "tp_moe_worker.py"), "cpu"]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=400)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    assert r.stdout.count("TP_MOE_WORKER_OK") == 2


@pytest.mark.parametrize("heads,kv", [(8, 2), (4, 4)])
def test_tp4_dense_decoder_matches_unsplit_model_with_replicated_kv_heads(heads, kv):
    """Four gloo ranks; with 2 KV heads each KV head is held by the two ranks whose query heads use it."""
    env = dict(os.environ, PYTHONPATH=ROOT, MASTER_ADDR="127.0.0.1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=4", "--master-addr", "127.0.0.1",
           "--master-port", str(29801 + kv), os.path.join(ROOT, "tests", "tp_dense_worker.py"), str(heads), str(kv)]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=400)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    assert r.stdout.count("TP_DENSE_WORKER_OK") == 4


@pytest.mark.parametrize("world", [2, 4])
def test_sequence_parallel_decoder_matches_allreduce_and_unsplit_models(world):
    """Residual stream sharded by rows between the tensor-parallel GEMMs (gloo ranks; uneven and empty shards)."""
    env = dict(os.environ, PYTHONPATH=ROOT, MASTER_ADDR="127.0.0.1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr",
           "127.0.0.1", "--master-port", str(29860 + world), os.path.join(ROOT, "tests", "sp_decoder_worker.py"), "cpu"]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    assert r.stdout.count("SP_DECODER_WORKER_OK") == world


def test_client_with_a_tensor_parallel_distributed_config():
    """The public client under torch.distributed.run: DistributedConfig(parallel.tp = world) builds each rank's shard;
    every rank makes the same calls and returns the tokens of the unsplit client."""
    env = dict(os.environ, PYTHONPATH=ROOT, MASTER_ADDR="127.0.0.1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29896", os.path.join(ROOT, "tests", "tp_client_worker.py")]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=400)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    assert r.stdout.count("TP_CLIENT_WORKER_OK") == 2


@pytest.mark.parametrize("world", [2, 3])
def test_engines_prefill_a_long_prompt_together(world):
    """``LLMEngine.add_request_context_parallel``: the ranks' engines split the prompt's full pages, exchange KV pages
    per layer, admit the request on the cached pages; tokens equal a single engine's, pools may differ per rank."""
    env = dict(os.environ, PYTHONPATH=ROOT, MASTER_ADDR="127.0.0.1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr",
           "127.0.0.1", "--master-port", str(29840 + world), os.path.join(ROOT, "tests", "cp_engine_worker.py")]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=400)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    assert r.stdout.count("CP_ENGINE_WORKER_OK") == world


@pytest.mark.parametrize("how", ["same", "other"])
def test_saguaro_draft_and_verify_on_different_ranks(how):
    """Rank 1 drafts with its own model, rank 0 verifies inside the serving engine: tokens equal plain greedy decoding
    of the target; with identical weights every draft is accepted, with another draft model some are rejected."""
    env = dict(os.environ, PYTHONPATH=ROOT, MASTER_ADDR="127.0.0.1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", str(29830 + (how == "same")), os.path.join(ROOT, "tests", "saguaro_worker.py"), how]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=400)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    assert r.stdout.count("SAGUARO_WORKER_OK") == 2


def test_vocab_parallel_sampling_from_top_k_candidates():
    """Three gloo ranks: every rank sends its 64 best (logit, index) pairs per row instead of its vocabulary shard;
    all ranks sample the same token, inside the global top-k of its row; top-1 and greedy rows give the argmax."""
    env = dict(os.environ, PYTHONPATH=ROOT, MASTER_ADDR="127.0.0.1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=3", "--master-addr", "127.0.0.1",
           "--master-port", "29893", os.path.join(ROOT, "tests", "tp_sample_worker.py")]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=400)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    assert r.stdout.count("TP_SAMPLE_WORKER_OK") == 3


@pytest.mark.parametrize("world", [2, 3])
def test_context_parallel_prefill_matches_single_rank_prefill(world):
    """Page-aligned prompt shards, KV pages exchanged after every layer's K/V write: same last-token logits and the
    same cache contents on every rank as one rank prefilling the whole prompts (gloo ranks)."""
    env = dict(os.environ, PYTHONPATH=ROOT, MASTER_ADDR="127.0.0.1")
    for mode in ("cpu", "cpu_zigzag"):      # contiguous shards, then two chunks per rank (balanced causal work)
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr",
               "127.0.0.1", "--master-port", str(29850 + world), os.path.join(ROOT, "tests", "cp_worker.py"), mode]
        r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
        assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
        assert r.stdout.count("CP_WORKER_OK") == world


def test_lockstep_engines_with_expert_parallel_moe_match_unsplit_engine():
    """Two serving engines, each with its own requests, share the expert-parallel MoE; outputs equal the plain engine's."""
    env = dict(os.environ, PYTHONPATH=ROOT, MASTER_ADDR="127.0.0.1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29798", os.path.join(ROOT, "tests", "ep_engine_worker.py"), "cpu"]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=400)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    assert r.stdout.count("EP_ENGINE_WORKER_OK") == 2


def test_nvlink_counter_reader_against_a_fake_nvml(monkeypatch):
    """The NVLink byte probe only READS the driver's throughput counters; here against a fake NVML."""
    import types
    import pynvml
    from gllm_b200.parallel import nvlink_probe as P

    calls = []

    def fake_get(handle, fields):
        calls.append(list(fields))
        vals = []
        for fid, scope in fields:
            v = types.SimpleNamespace(nvmlReturn=0, value=types.SimpleNamespace(ullVal=1000 * fid + 7))
            vals.append(v)
        return vals

    monkeypatch.setattr(pynvml, "nvmlDeviceGetFieldValues", fake_get)
    tx, rx = P.read_nvlink_kib(object())
    assert (tx, rx) == (138007, 139007)
    assert calls == [[(138, 0xFFFFFFFF), (139, 0xFFFFFFFF)]]

    def failing(handle, fields):
        return [types.SimpleNamespace(nvmlReturn=3, value=types.SimpleNamespace(ullVal=0)) for _ in fields]

    monkeypatch.setattr(pynvml, "nvmlDeviceGetFieldValues", failing)
    assert P.read_nvlink_kib(object()) is None


@pytest.mark.parametrize("world", [2, 3])
def test_sequence_parallel_block_allgather_gemm_reduce_scatter_on_gloo(world):
    """Row-sharded activations: all-gather -> column-parallel GEMM -> row-parallel GEMM -> reduce-scatter (the unfused
    forms on gloo ranks; the fused kernels run the same worker on GPUs)."""
    env = dict(os.environ, PYTHONPATH=ROOT, MASTER_ADDR="127.0.0.1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr",
           "127.0.0.1", "--master-port", str(29860 + world), os.path.join(ROOT, "tests", "sp_worker.py"), "cpu"]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=400)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    assert r.stdout.count("SP_WORKER_OK") == world


def test_comm_config_selects_the_all_reduce_form():
    from gllm_b200.parallel.config import CommAlgorithm, CommConfig
    from gllm_b200.parallel.tensor_parallel import mode_for_comm_config
    assert mode_for_comm_config(CommConfig()) == "auto"
    assert mode_for_comm_config(CommConfig(algorithm=CommAlgorithm.HARDWARE_REDUCE)) == "pull"
    assert mode_for_comm_config(CommConfig(algorithm=CommAlgorithm.DIRECT)) == "ll_p2p"
    assert mode_for_comm_config(CommConfig(algorithm=CommAlgorithm.RING)) == "nccl"
    assert mode_for_comm_config(CommConfig(overlap="prefer_isolated")) == "nccl"
