"""Continuous-batching scheduler against a fake backend (token = previous + 1), and against the CPU Llama engine."""

import pytest
import torch

from mfq_b200.engine.scheduler import (BackendFailure, ContinuousBatchScheduler, DeadlineExceeded, QueueFull, QueueTimeout,
                                       Request, SamplingParams)


class FakeBackend:
    """Every sequence continues with last+1; KV memory is a token budget in 16-token pages."""

    def __init__(self, max_batch=4, pages=64, fail_prefill_for=(), fail_decode_at=None):
        self.max_batch, self.pages_total = max_batch, pages
        self.rows: dict[int, list[int]] = {}
        self.fail_prefill_for, self.fail_decode_at = set(fail_prefill_for), fail_decode_at
        self.decodes = 0

    def _pages(self, n):
        return (n + 15) // 16

    def free_tokens(self):
        return (self.pages_total - sum(self._pages(len(t) + 1) for t in self.rows.values())) * 16

    def tokens_needed(self, tokens):
        return self._pages(tokens) * 16

    def prefill(self, row, tokens, params):
        if tokens[0] in self.fail_prefill_for:
            raise ValueError("bad prompt")
        if self._pages(len(tokens) + 1) * 16 > self.free_tokens():
            raise MemoryError
        self.rows[row] = list(tokens)
        nxt = tokens[-1] + 1
        self.rows[row].append(nxt)
        return nxt

    def can_grow(self, row):
        grow = self._pages(len(self.rows[row]) + 1) - self._pages(len(self.rows[row]))
        return grow * 16 <= self.free_tokens()

    def decode(self, rows):
        self.decodes += 1
        if self.fail_decode_at is not None and self.decodes >= self.fail_decode_at:
            raise RuntimeError("device lost")
        out = {}
        for r in rows:
            nxt = self.rows[r][-1] + 1
            self.rows[r].append(nxt)
            out[r] = nxt
        return out

    def release(self, row):
        self.rows.pop(row, None)


def collect(req):
    events = []
    req.on_event = events.append
    return events


def test_batched_generation_and_priorities():
    be = FakeBackend(max_batch=2)
    s = ContinuousBatchScheduler(be)
    reqs = [Request([100 * i], SamplingParams(max_tokens=5), priority=(5 if i == 3 else 0)) for i in range(1, 5)]
    evs = [collect(r) for r in reqs]
    for r in reqs:
        s.submit(r)
    s.run_until_idle()
    for i, r in enumerate(reqs, 1):
        assert r.generated == [100 * i + j for j in range(1, 6)] and r.finish_reason == "length"
        assert [e.kind for e in evs[i - 1]].count("token") == 5 and evs[i - 1][-1].kind == "completed"
    assert reqs[2].start_time <= min(r.start_time for r in reqs if r is not reqs[2])  # priority 5 ran first
    assert s.stats.completed == 4 and not be.rows


def test_stop_token_and_cancel():
    s = ContinuousBatchScheduler(FakeBackend())
    a = Request([10], SamplingParams(max_tokens=50, stop_token_ids=(13,)))
    b = Request([20], SamplingParams(max_tokens=50))
    s.submit(a)
    s.submit(b)
    for _ in range(4):
        s.step()
    assert s.cancel(b.id)
    s.run_until_idle()
    assert a.generated == [11, 12, 13] and a.finish_reason == "stop" and b.finish_reason == "cancelled"


def test_queue_full_timeout_and_deadline():
    t = [0.0]
    be = FakeBackend(max_batch=1)
    s = ContinuousBatchScheduler(be, max_queue=2, queue_timeout=5.0, clock=lambda: t[0])
    long_req = Request([1], SamplingParams(max_tokens=1000))
    s.submit(long_req)
    s.step()
    w1, w2 = Request([2], SamplingParams(max_tokens=3)), Request([3], SamplingParams(max_tokens=3), timeout_seconds=2.0)
    s.submit(w1)
    s.submit(w2)
    with pytest.raises(QueueFull):
        s.submit(Request([4]))
    t[0] = 3.0
    s.step()
    assert isinstance(w2.error, DeadlineExceeded) and w2.finish_reason == "runtime_deadline_exceeded"
    t[0] = 6.0
    s.step()
    assert isinstance(w1.error, QueueTimeout)
    assert not long_req.finished


def test_retraction_and_replay_under_kv_pressure():
    be = FakeBackend(max_batch=4, pages=6)
    s = ContinuousBatchScheduler(be)
    reqs = [Request(list(range(1000 * i, 1000 * i + 10)), SamplingParams(max_tokens=40)) for i in range(1, 4)]
    for r in reqs:
        s.submit(r)
    s.run_until_idle()
    assert s.stats.retractions >= 1
    for i, r in enumerate(reqs, 1):
        assert r.finish_reason == "length"
        assert r.generated == [1000 * i + 10 + j for j in range(40)]  # replay after retraction reproduces the stream


def test_prefill_failure_is_isolated_and_decode_failure_poisons():
    be = FakeBackend(fail_prefill_for={7})
    s = ContinuousBatchScheduler(be)
    bad, good = Request([7], SamplingParams(max_tokens=3)), Request([8], SamplingParams(max_tokens=3))
    s.submit(bad)
    s.submit(good)
    s.run_until_idle()
    assert bad.finish_reason == "error" and good.generated == [9, 10, 11] and s.healthy
    be2 = FakeBackend(fail_decode_at=2)
    s2 = ContinuousBatchScheduler(be2)
    r1, r2 = Request([1], SamplingParams(max_tokens=9)), Request([5], SamplingParams(max_tokens=9))
    s2.submit(r1)
    s2.submit(r2)
    s2.run_until_idle()
    assert not s2.healthy and isinstance(r1.error, BackendFailure) and isinstance(r2.error, BackendFailure)
    with pytest.raises(BackendFailure):
        s2.submit(Request([1]))


def test_scheduler_drives_the_cpu_engine():
    from mfq_b200.engine.llm_engine import LLMEngine
    from mfq_b200.models.llama import LlamaConfig, LlamaModel, LlamaWeights
    cfg = LlamaConfig.tiny()
    w = LlamaWeights.random_init(cfg, "cpu", seed=5, std=0.05)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=torch.Generator().manual_seed(n)).tolist() for n in (9, 21, 14)]
    static = LLMEngine(LlamaModel(cfg, w), max_batch=4, max_seq_len=64, device="cpu")
    want = [static.generate([torch.tensor(p)], 6).tokens[0].tolist() for p in prompts]
    eng = LLMEngine(LlamaModel(cfg, w), max_batch=2, max_seq_len=64, device="cpu")
    s = ContinuousBatchScheduler(eng)
    reqs = [Request(p, SamplingParams(max_tokens=6)) for p in prompts]
    for r in reqs:
        s.submit(r)
    s.run_until_idle()
    assert [r.generated for r in reqs] == want
    assert eng.cache.allocator.free_pages == eng.cache.num_pages - 1


def test_stochastic_sampling_is_seeded_cpu():
    from mfq_b200.engine.llm_engine import LLMEngine
    from mfq_b200.models.llama import LlamaConfig, LlamaModel, LlamaWeights
    cfg = LlamaConfig.tiny()
    w = LlamaWeights.random_init(cfg, "cpu", seed=5, std=0.05)
    outs = []
    for _ in range(2):
        eng = LLMEngine(LlamaModel(cfg, w), max_batch=1, max_seq_len=64, device="cpu")
        s = ContinuousBatchScheduler(eng)
        r = Request([5, 6, 7], SamplingParams(max_tokens=8, temperature=1.0, top_k=50, top_p=0.9, seed=1234))
        s.submit(r)
        s.run_until_idle()
        outs.append(r.generated)
    assert outs[0] == outs[1] and len(set(outs[0])) > 1
