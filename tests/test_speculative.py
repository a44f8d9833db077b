import torch

from gllm_b200.models.config import preset
from gllm_b200.models.decoder import DecoderModel
from gllm_b200.models.weights import RandomWeights
from gllm_b200.speculative import (AcceptanceController, DraftAdapter, EagleHead, KvOp, MtpExecutor, MtpHead, NgramIndex,
                                   SelfSpeculativeDecoder, SpecDecodingState, SpecMode, SpecTree, SpeculationCache,
                                   generate_kv_commit_instructions, parse_step_tokens, tree_attention_mask_csr,
                                   tree_attention_mask_dense, verify_greedy, verify_stochastic, verify_tree_greedy)


def test_ngram_index_and_tree_mask():
    ix = NgramIndex(2, 3)
    ix.extend([1, 2, 3, 4, 9, 1, 2, 3])
    assert ix.lookup(3) == [[4, 9, 1]]
    ix.extend([7]); assert ix.lookup(2) == []
    t = SpecTree.build([5, 6, 7], branches=[[5, 8], [9]])
    assert t.tokens() == [5, 6, 7, 8, 9] and t.depths() == [0, 1, 2, 1, 0]
    rp, ci = tree_attention_mask_csr(t)
    assert rp == [0, 1, 3, 6, 8, 9] and ci[3:6] == [0, 1, 2] and ci[6:8] == [0, 3]
    m = tree_attention_mask_dense(t)
    assert m[3].tolist() == [True, False, False, True, False] and sorted(map(tuple, t.paths())) == [(0, 1, 2), (0, 3), (4,)]


def test_verification_rules_and_kv_commit():
    assert verify_greedy([4, 5, 6], [4, 5, 9, 1]) == (2, 9) and verify_greedy([4], [4, 7]) == (1, 7) and verify_greedy([], [3]) == (0, 3)
    t = SpecTree.build([5, 6, 7], branches=[[5, 8]])
    acc, nxt = verify_tree_greedy(t, target_argmax_at_node=[8, 0, 0, 2], root_argmax=5)
    assert acc == [0, 3] and nxt == 2
    ins = generate_kv_commit_instructions(100, node_slots=[100, 101, 102, 103], accepted_nodes=acc)
    assert [(i.op, i.src_slot, i.dst_slot) for i in ins[:2]] == [(KvOp.KEEP, 100, 100), (KvOp.MOVE, 103, 101)]
    assert sorted(i.src_slot for i in ins if i.op == KvOp.DROP) == [101, 102]
    # rejection sampling keeps the target distribution
    g = torch.Generator().manual_seed(0)
    p = torch.tensor([[0.7, 0.2, 0.1], [0.1, 0.1, 0.8]])
    q = torch.tensor([[0.2, 0.5, 0.3]])
    counts = torch.zeros(3)
    for _ in range(4000):
        d = int(torch.multinomial(q[0], 1, generator=g))
        n, tok = verify_stochastic([d], q, p, g)
        counts[d if n == 1 else tok] += 1
    assert (counts / counts.sum() - p[0]).abs().max() < 0.03


def test_controller_state_heads_and_mtp():
    c = AcceptanceController()
    for _ in range(30):
        c.update(8, 8)
    assert c.draft_len() == c.max_draft
    for _ in range(40):
        c.update(0, 4)
    assert c.draft_len() == 0
    s = SpecDecodingState(SpecMode.NGRAM)
    assert s.should_speculate(4) and not s.should_speculate(64) and not SpecDecodingState().should_speculate(1)
    s.record(4, 2); s.record(4, 4)
    assert s.acceptance_rate == 0.75 and s.tokens_per_step == 4.0
    H, V = 32, 50
    emb, head, norm = torch.randn(V, H), torch.randn(V, H), torch.ones(H)
    hid = torch.randn(3, H)
    assert DraftAdapter(norm, head).draft_token(hid).shape == (3,)
    eg = EagleHead(H, emb, head, norm)
    d = eg.draft(hid, torch.tensor([1, 2, 3]), depth=3)
    assert len(d) == 3 and d[0].shape == (3,)
    assert MtpHead(H, emb, head).logits(hid, torch.tensor([1, 2, 3])).shape == (3, V)
    sc = SpeculationCache(2)
    sc.put(1, [4, 5], 10, 0); sc.put(2, [6], 3, 0); sc.put(3, [7], 3, 0)
    assert sc.take(1, 10) is None and sc.take(2, 4) is None and sc.take(3, 3).tokens == [7]
    outs = parse_step_tokens([9, 1, 2, 8, 3, 4], depth=2)
    assert outs[1].main_token == 8 and outs[1].candidates == [3, 4]
    v = MtpExecutor(2).verify([1, 2], [1, 5, 0])
    assert (v.accepted, v.next_token, v.rollback_tokens) == (1, 5, 1)


def test_self_speculative_decoding_equals_greedy():
    cfg = preset("tiny-llama")
    src = RandomWeights(cfg, "cpu", torch.float32, seed=11, std=0.05)
    model = DecoderModel(cfg, src, device="cpu", dtype=torch.float32, max_positions=512)
    prompt = [3, 17, 29, 41, 3, 17, 29, 41, 3, 17, 29, 41, 3, 17]
    plain = SelfSpeculativeDecoder(model, state=SpecDecodingState(SpecMode.OFF)).generate(prompt, 24)
    spec = SelfSpeculativeDecoder(model, state=SpecDecodingState(SpecMode.NGRAM))
    got = spec.generate(prompt, 24)
    assert got == plain and len(got) == 24
    # an oracle drafter that always proposes the true continuation is fully accepted
    full = prompt + plain
    oracle = SelfSpeculativeDecoder(model, draft_fn=lambda toks, k: full[len(toks):len(toks) + k])
    assert oracle.generate(prompt, 24) == plain and oracle.state.acceptance_rate == 1.0 and oracle.state.tokens_per_step > 2
