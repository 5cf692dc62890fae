"""Session snapshots (CPU path): a follow-up turn restores the conversation's KV pages and recurrent state."""

import pytest
import torch

from mfq_b200.engine.llm_engine import LLMEngine
from mfq_b200.engine.session_cache import SessionSnapshotCache
from mfq_b200.models.hybrid import HybridConfig, HybridModel, HybridWeights, init_hybrid_weights
from mfq_b200.models.llama import LlamaConfig, LlamaModel, LlamaWeights


def _model(kind):
    if kind == "llama":
        cfg = LlamaConfig.tiny()
        return cfg, LlamaModel(cfg, LlamaWeights.random_init(cfg, "cpu", seed=2, std=0.05))
    cfg = HybridConfig.tiny()
    return cfg, HybridModel(cfg, HybridWeights.from_tensors(cfg, init_hybrid_weights(cfg, seed=3, std=0.05), "cpu"))


@pytest.mark.parametrize("kind", ["llama", "hybrid"])
def test_followup_turn_restores_snapshot(kind):
    cfg, model = _model(kind)
    g = torch.Generator().manual_seed(1)
    turn1 = torch.randint(0, cfg.vocab_size, (41,), generator=g)
    plain = LLMEngine(model, max_batch=1, max_seq_len=128, device="cpu")
    reply = plain.generate([turn1], 6).tokens[0]
    turn2 = torch.cat([turn1, reply, torch.randint(0, cfg.vocab_size, (11,), generator=g)]).to(torch.int32)
    plain.release(0)
    want = plain.generate([turn2], 5).tokens[0].tolist()

    eng = LLMEngine(model, max_batch=1, max_seq_len=128, device="cpu")
    eng.session_cache = SessionSnapshotCache(budget_bytes=64 << 20)
    assert eng.generate([turn1], 6).tokens[0].tolist() == reply.tolist()
    # the cache holds the prompt and all but the last sampled token
    covered = torch.cat([turn1, reply[:-1]]).tolist()
    assert int(eng.seq_lens[0]) == len(covered)
    eng.session_cache.save(eng, 0, "chat-1", covered)
    eng.release(0)
    tok = eng.prefill(0, turn2, session="chat-1")
    assert eng.session_cache.stats["restored"] == 1 and eng.session_cache.stats["tokens_skipped"] == len(covered)
    eng.grow(0, len(turn2) + 8)
    got = [tok]
    for _ in range(4):
        eng.decode_step(1)
        got.append(int(eng.sampled[0]))
    assert got == want
    # an edited conversation drops the snapshot
    eng.release(0)
    edited = turn2.clone()
    edited[3] = (edited[3] + 1) % cfg.vocab_size
    eng.prefill(0, edited, session="chat-1")
    assert eng.session_cache.stats["dropped_mismatch"] == 1 and "chat-1" not in eng.session_cache.entries


def test_lru_budget():
    cfg, model = _model("llama")
    eng = LLMEngine(model, max_batch=1, max_seq_len=128, device="cpu")
    p = torch.randint(0, cfg.vocab_size, (40,), generator=torch.Generator().manual_seed(0))
    eng.prefill(0, p)
    one = SessionSnapshotCache()
    one.save(eng, 0, "a", p.tolist())
    size = one.bytes
    sc = SessionSnapshotCache(budget_bytes=2 * size)
    for name in "abc":
        sc.save(eng, 0, name, p.tolist())
    assert list(sc.entries) == ["b", "c"] and sc.stats["evicted"] == 1 and sc.bytes == 2 * size


def test_scheduler_saves_and_restores_by_session():
    from mfq_b200.engine.scheduler import ContinuousBatchScheduler, Request, SamplingParams
    cfg, model = _model("hybrid")
    eng = LLMEngine(model, max_batch=2, max_seq_len=128, device="cpu")
    eng.session_cache = SessionSnapshotCache()
    sched = ContinuousBatchScheduler(eng)
    g = torch.Generator().manual_seed(4)
    turn1 = torch.randint(0, cfg.vocab_size, (30,), generator=g).tolist()
    r1 = Request(turn1, SamplingParams(max_tokens=5), session="s")
    sched.submit(r1)
    sched.run_until_idle()
    assert eng.session_cache.stats["saved"] == 1
    assert eng.session_cache.entries["s"].tokens == (turn1 + r1.generated)[:-1]
    turn2 = turn1 + r1.generated + torch.randint(0, cfg.vocab_size, (7,), generator=g).tolist()
    r2 = Request(turn2, SamplingParams(max_tokens=4), session="s")
    sched.submit(r2)
    sched.run_until_idle()
    assert eng.session_cache.stats["restored"] == 1
    fresh = LLMEngine(model, max_batch=2, max_seq_len=128, device="cpu")
    assert fresh.generate([torch.tensor(turn2, dtype=torch.int32)], 4).tokens[0].tolist() == r2.generated
