"""Lockstep serving: the leader's scheduler drives a follower engine through the command log (threads + HashStore)."""

import threading

import pytest
import torch
import torch.distributed as dist

from mfq_b200.engine.llm_engine import LLMEngine
from mfq_b200.engine.scheduler import BackendFailure, ContinuousBatchScheduler, Request, SamplingParams
from mfq_b200.models.llama import LlamaConfig, LlamaModel, LlamaWeights
from mfq_b200.parallel.spmd import CommandLog, LeaderBackend, follower_loop


def _engine():
    cfg = LlamaConfig.tiny()
    return LLMEngine(LlamaModel(cfg, LlamaWeights.random_init(cfg, "cpu", seed=3)), max_batch=4, max_seq_len=96, device="cpu")


def test_follower_mirrors_every_state_change():
    store = dist.HashStore()
    lead, follow = _engine(), _engine()
    calls = []
    for name in ("prefill", "decode", "release"):
        real = getattr(follow, name)
        setattr(follow, name, (lambda n, f: lambda *a, **k: (calls.append(n), f(*a, **k))[1])(name, real))
    ended = {}
    t = threading.Thread(target=lambda: ended.setdefault("why", follower_loop(follow, CommandLog(store, 1, 2), 0.05)))
    t.start()
    backend = LeaderBackend(lead, CommandLog(store, 0, 2))
    sched = ContinuousBatchScheduler(backend, max_queue=8)
    done = []
    reqs = [Request(list(range(5 + i, 25 + 3 * i)), SamplingParams(max_tokens=6, temperature=0.7 if i == 1 else 0.0, seed=11),
                    on_event=lambda ev, i=i: done.append(i) if ev.kind == "completed" else None) for i in range(3)]
    for r in reqs:
        sched.submit(r)
    for _ in range(200):
        if not sched.step() and sched.idle:
            break
    assert sorted(done) == [0, 1, 2] and all(len(r.generated) >= 1 for r in reqs)
    # a row that is still open on both sides: same pages, same lengths, same next token
    row_ids = list(range(40, 60))
    first = backend.prefill(0, row_ids, None)
    backend.decode([0])
    backend.shutdown_followers()
    t.join(timeout=30)
    assert ended["why"] == "shutdown" and {"prefill", "decode", "release"} <= set(calls)
    assert follow.row_len == lead.row_len and follow.row_seq == lead.row_seq
    assert torch.equal(follow.sampled, lead.sampled)
    assert torch.equal(follow.cache.block_table, lead.cache.block_table)
    assert follow.cache.allocator.free_pages == lead.cache.allocator.free_pages
    kv_l, kv_f = lead.cache.layer(0), follow.cache.layer(0)
    assert torch.equal(kv_l.k.view(torch.uint8), kv_f.k.view(torch.uint8))


def test_follower_failure_reaches_the_leader_and_lost_leader_ends_the_follower():
    store = dist.HashStore()
    lead, follow = _engine(), _engine()

    def boom(*a, **k):
        raise RuntimeError("device status word set")
    follow.decode = boom
    ended = {}
    t = threading.Thread(target=lambda: ended.setdefault("why", follower_loop(follow, CommandLog(store, 1, 2), 0.05)))
    t.start()
    backend = LeaderBackend(lead, CommandLog(store, 0, 2))
    backend.prefill(0, list(range(3, 20)), None)
    backend.decode([0])
    t.join(timeout=30)
    assert ended["why"] == "error"
    with pytest.raises(BackendFailure, match="rank.*1.*device status word"):
        backend.decode([0])
    # a follower whose leader stopped beating gives up instead of waiting forever
    store2 = dist.HashStore()
    log = CommandLog(store2, 0, 2)
    log.beat()
    store2.set("spmd/leader_beat", "1.0")  # long ago
    assert follower_loop(_engine(), CommandLog(store2, 1, 2), 0.05, leader_timeout=1.0) == "leader_lost"
