"""Host scheduler (C++): allocator, prefix index, decode-first batching, chunked prefill, preemption."""
import numpy as np
import pytest

from gllm_b200 import scheduler as S


def _params(n=4, eos=()):
    return S.SamplingParams(temperature=0.0, top_k=0, top_p=1.0, max_new_tokens=n, eos_ids=list(eos))


def test_block_allocator_fifo_and_refcounts():
    a = S.BlockAllocator(4)
    p = [a.allocate() for _ in range(4)]
    assert p == [0, 1, 2, 3] and a.allocate() == -1
    a.retain(1)
    assert not a.release(1) and a.release(1)
    assert a.num_free == 1 and a.allocate() == 1          # FIFO reuse
    with pytest.raises(RuntimeError):
        a.release(1) and a.release(1) and a.release(1)


def test_prefix_index_full_pages_only_and_lru_evict():
    a = S.BlockAllocator(8)
    idx = S.PrefixIndex(a, 4)
    toks = list(range(10))
    pages = [a.allocate() for _ in range(3)]
    idx.insert(toks, pages[:2])                           # two full pages cached
    n, got = idx.find_longest_prefix(toks + [99])
    assert n == 8 and got == pages[:2]
    n, got = idx.find_longest_prefix([0, 1, 2, 3, 7, 7, 7, 7])
    assert n == 4 and got == pages[:1]
    assert idx.find_longest_prefix([5, 5, 5, 5])[0] == 0
    for p in pages:
        a.release(p)                                      # only the cache holds pages 0,1 now
    assert a.num_free == 6 and idx.cached_pages == 2
    assert idx.evict(1) == 1 and idx.cached_pages == 1    # leaf (second page) goes first
    assert idx.find_longest_prefix(toks)[0] == 4


def test_decode_first_then_prefill_backfill_and_completion():
    cfg = S.PolicyConfig()
    cfg.max_batch_tokens, cfg.prefill_chunk, cfg.min_prefill_chunk = 32, 16, 1
    b = S.ContinuousBatcher(64, 4, 8, 32, cfg)
    b.add_request(1, list(range(100, 110)), _params(3))
    b.add_request(2, list(range(200, 240)), _params(2))
    plan = b.schedule()
    assert plan.num_decode == 0 and plan.num_prefill_seqs == 2
    assert list(plan.pf_q_len) == [10, 16]                # request 2 is chunked to the 16-token cap
    assert plan.prefill[0].last and not plan.prefill[1].last
    b.commit(plan, np.zeros(8, np.int32), np.array([7], np.int32))
    plan = b.schedule()                                    # request 1 decodes, request 2 continues prefill
    assert plan.num_decode == 1 and plan.num_prefill_seqs == 1
    slot = b.state_of(1)["slot"]
    assert plan.dec_tokens[slot] == 7 and plan.dec_positions[slot] == 10 and plan.dec_ctx_lens[slot] == 11
    bt = b.block_table_of(1)
    assert plan.dec_slot_mapping[slot] == bt[10 // 4] * 4 + 10 % 4
    dec = np.zeros(8, np.int32); dec[slot] = 8
    b.commit(plan, dec, np.zeros(0, np.int32))
    done = []
    for _ in range(10):
        plan = b.schedule()
        if plan.idle:
            break
        dec = np.full(8, 9, np.int32)
        b.commit(plan, dec, np.full(plan.num_sampled_prefill, 5, np.int32))
        done += b.pop_finished()
    ids = {f.id: f for f in done}
    assert list(ids[1].tokens) == [7, 8, 9] and ids[1].finish == 2
    assert list(ids[2].tokens) == [5, 9] and b.num_running == 0 and b.num_waiting == 0


def test_prefix_reuse_binds_shared_pages_and_leaves_one_token():
    cfg = S.PolicyConfig()
    cfg.max_batch_tokens, cfg.min_prefill_chunk = 256, 1
    b = S.ContinuousBatcher(64, 4, 8, 32, cfg)
    shared = list(range(16))
    b.add_request(1, shared + [50, 51], _params(1))
    plan = b.schedule()
    b.commit(plan, np.zeros(8, np.int32), np.array([1], np.int32))
    assert b.pop_finished()[0].cached_prefix == 0 and b.cached_pages == 4
    b.add_request(2, shared + [60], _params(1))
    b.add_request(3, shared, _params(1))                   # whole prompt cached: still computes >= 1 token
    plan = b.schedule()
    assert list(plan.pf_q_len) == [1, 4] and list(plan.pf_positions[:1]) == [16]
    assert list(plan.pf_ctx_lens) == [17, 16]
    bt2, bt3 = b.block_table_of(2), b.block_table_of(3)
    assert bt2[:4] == bt3[:3] + [bt2[3]] and bt2[:3] == bt3[:3]
    assert b.prefix_hits == 2
    b.commit(plan, np.zeros(8, np.int32), np.array([1, 1], np.int32))
    fin = {f.id: f for f in b.pop_finished()}
    assert fin[2].cached_prefix == 16 and fin[3].cached_prefix == 12


def test_eos_stops_and_length_guard():
    b = S.ContinuousBatcher(16, 4, 4, 8, S.PolicyConfig())
    with pytest.raises(Exception):
        b.add_request(1, list(range(30)), _params(10))     # 40 tokens > 8 blocks * 4
    b.add_request(2, [1, 2, 3], _params(10, eos=[42]))
    plan = b.schedule()
    b.commit(plan, np.zeros(4, np.int32), np.array([42], np.int32))
    f = b.pop_finished()
    assert len(f) == 1 and f[0].finish == 1 and list(f[0].tokens) == [42]
    assert b.num_free_pages + b.cached_pages == 16


def test_oom_preempts_youngest_and_recovers():
    cfg = S.PolicyConfig()
    cfg.max_batch_tokens, cfg.min_prefill_chunk, cfg.watermark_pages = 64, 1, 0
    cfg.enable_prefix_cache = False
    b = S.ContinuousBatcher(4, 4, 4, 8, cfg)              # 16 tokens of KV in total
    b.add_request(1, list(range(7)), _params(8))
    b.add_request(2, list(range(10, 17)), _params(8))
    plan = b.schedule()
    assert plan.num_prefill_seqs == 2
    b.commit(plan, np.zeros(4, np.int32), np.array([1, 1], np.int32))
    finished, preempted = [], 0
    for _ in range(60):
        plan = b.schedule()
        preempted += len(plan.preempted)
        if plan.idle:
            break
        b.commit(plan, np.full(4, 3, np.int32), np.full(plan.num_sampled_prefill, 3, np.int32))
        finished += b.pop_finished()
    assert preempted >= 1 and sorted(f.id for f in finished) == [1, 2]
    assert all(len(f.tokens) == 8 for f in finished)
    assert b.num_free_pages == 4


def test_policy_thresholds():
    cfg = S.PolicyConfig()
    cfg.max_batch_size = 32
    st = S.SystemState()
    assert S.policy_decide(cfg, st).max_batch_size == 32
    st.memory_pressure = 0.95
    d = S.policy_decide(cfg, st)
    assert not d.admit_new_prefill and d.force_swap_out_count == 3
    st.memory_pressure, st.kv_fragmentation = 0.1, 0.6
    d = S.policy_decide(cfg, st)
    assert not d.admit_new_prefill and d.force_swap_out_count == 1
    st.kv_fragmentation, st.attention_sparsity = 0.0, 0.8
    assert S.policy_decide(cfg, st).max_batch_size == int(32 * 0.6)
    st.attention_sparsity, st.logits_entropy, st.running = 0.0, 9.0, 5
    assert S.policy_decide(cfg, st).max_batch_size == 5


def test_rollback_for_speculative_decode():
    cfg = S.PolicyConfig(); cfg.min_prefill_chunk = 1
    b = S.ContinuousBatcher(16, 4, 4, 8, cfg)
    b.add_request(1, [1, 2, 3], _params(20))
    plan = b.schedule(); b.commit(plan, np.zeros(4, np.int32), np.array([9], np.int32))
    for _ in range(6):
        plan = b.schedule(); b.commit(plan, np.full(4, 9, np.int32), np.zeros(0, np.int32))
    st = b.state_of(1)
    assert st["num_tokens"] == 10 and st["pages"] == 3
    assert b.rollback(1, 4)
    st = b.state_of(1)
    assert st["num_tokens"] == 6 and st["num_computed"] == 5 and st["pages"] == 2
    assert b.append_tokens(1, [4, 5]) and b.state_of(1)["num_tokens"] == 8
