"""Session snapshot: a fresh engine that loaded the snapshot reuses the conversation's KV pages (prefix hit) and
produces the same continuation as the engine that computed them."""
import torch

from gllm_b200.engine.checkpoint import load_sessions, save_sessions
from gllm_b200.engine.executor import EngineConfig, LLMEngine
from gllm_b200.models.config import preset
from gllm_b200.models.decoder import DecoderModel
from gllm_b200.models.weights import RandomWeights


def _engine():
    cfg = preset("tiny-qwen3")
    src = RandomWeights(cfg, "cpu", torch.float32, seed=7, std=0.05)
    m = DecoderModel(cfg, src, device="cpu", dtype=torch.float32, max_positions=256)
    return LLMEngine(m, EngineConfig(max_num_seqs=4, max_model_len=256, max_batch_tokens=128, num_pages=64))


def test_snapshot_and_restore_session(tmp_path):
    turn1 = [(5 * i + 1) % 1000 for i in range(50)]
    e1 = _engine()
    rid = e1.submit(turn1, max_tokens=14, temperature=0.0, eos_ids=[], session_id="chat-1")
    e1.run_until_done()
    out1 = e1.results[rid].token_ids
    assert e1.batcher.session_ids() == ["chat-1"] and e1.batcher.session_cached_tokens("chat-1") >= 48
    path = str(tmp_path / "sessions.pt")
    saved = save_sessions(e1, path)
    assert saved["chat-1"] == 48                      # 63 computed tokens -> 3 whole pages
    turn2 = turn1 + out1 + [7, 8, 9]
    rid2 = e1.submit(turn2, max_tokens=6, temperature=0.0, eos_ids=[], session_id="chat-1")
    e1.run_until_done()
    want = e1.results[rid2]
    # a brand-new engine: without the snapshot no prefix is cached; with it the history pages are reused
    cold = _engine()
    r = cold.submit(turn2, max_tokens=6, temperature=0.0, eos_ids=[])
    cold.run_until_done()
    assert cold.results[r].telemetry.cached_prefix_tokens == 0 and cold.results[r].token_ids == want.token_ids
    warm = _engine()
    assert load_sessions(warm, path) == {"chat-1": 48}
    assert warm.batcher.session_cached_tokens("chat-1") == 48
    r = warm.submit(turn2, max_tokens=6, temperature=0.0, eos_ids=[], session_id="chat-1")
    warm.run_until_done()
    res = warm.results[r]
    assert res.telemetry.cached_prefix_tokens == 48 and res.token_ids == want.token_ids
    assert load_sessions(warm, path) == {"chat-1": 48}      # idempotent: pages already there are skipped
