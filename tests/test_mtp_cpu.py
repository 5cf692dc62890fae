"""MTP draft/verify decoding on the CPU reference path: lossless w.r.t. plain greedy decoding, acceptance bookkeeping."""

import pytest
import torch

from mfq_b200.engine.llm_engine import LLMEngine
from mfq_b200.engine.scheduler import ContinuousBatchScheduler, Request, SamplingParams
from mfq_b200.models.llama import LlamaConfig, LlamaModel, LlamaWeights
from mfq_b200.ops import mtp as mtp_ops


def _engine(k, max_batch=2, mtp=True, **kw):
    cfg = LlamaConfig.tiny()
    w = LlamaWeights.random_init(cfg, "cpu", seed=5, std=0.05, mtp=mtp)
    return cfg, LLMEngine(LlamaModel(cfg, w), max_batch=max_batch, max_seq_len=96, device="cpu", mtp_draft_tokens=k, **kw)


def _agree(a, b):
    """Length of the common prefix, as a fraction."""
    n = 0
    while n < len(a) and a[n] == b[n]:
        n += 1
    return n / len(a)


@pytest.mark.parametrize("k", [1, 3])
def test_mtp_generation_matches_plain_greedy(k):
    cfg, eng = _engine(k)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=torch.Generator().manual_seed(n)) for n in (9, 14)]
    plain = eng.generate(prompts, 12).tokens
    for r in range(2):
        eng.release(r)
    spec = eng.generate(prompts, 12, use_mtp=True).tokens
    # the verify pass batches K+1 positions, so float summation order differs slightly from one-token decode;
    # near-ties of a random-init model may flip late in the sequence
    assert min(_agree(plain[r].tolist(), spec[r].tolist()) for r in range(2)) >= 0.75
    st = eng.mtp_stats()
    assert st["drafted"] > 0 and 0.0 <= st["acceptance_rate"] <= 1.0


def test_oracle_drafts_are_all_accepted():
    cfg, eng = _engine(3, max_batch=1)
    prompt = torch.randint(0, cfg.vocab_size, (11,), generator=torch.Generator().manual_seed(1))
    truth = eng.generate([prompt], 8).tokens[0].tolist()
    eng.release(0)
    first = eng.prefill(0, prompt)
    eng.grow(0, 40)
    assert first == truth[0]
    eng.draft[0] = torch.tensor(truth[1:4], dtype=torch.int32)
    eng.active.fill_(1)
    eng.mtp_step(1)
    n = int(eng.n_out[0])
    got = eng.out_tokens[0, :n].tolist()
    assert got == truth[1 : 1 + n]
    assert n >= 3  # all three drafts confirmed (+ the bonus token) unless a float near-tie intervened
    assert int(eng.seq_lens[0]) == 11 + n and int(eng.sampled[0]) == got[-1]
    # a wrong first draft confirms exactly one token
    eng.draft[0] = torch.tensor([(truth[1 + n] + 1) % cfg.vocab_size, 0, 0], dtype=torch.int32)
    before = int(eng.seq_lens[0])
    eng.mtp_step(1)
    assert int(eng.n_out[0]) == 1 and int(eng.seq_lens[0]) == before + 1


def test_accept_bookkeeping():
    draft = torch.tensor([[5, 6, 7], [5, 9, 7], [1, 2, 3]], dtype=torch.int32)
    targets = torch.tensor([[5, 6, 7, 8], [5, 6, 7, 8], [4, 2, 3, 9]], dtype=torch.int32).reshape(-1)
    head_next = torch.arange(100, 112, dtype=torch.int32)
    sampled, seq = torch.zeros(3, dtype=torch.int32), torch.tensor([10, 20, 30], dtype=torch.int32)
    out, n_out, arow = torch.full((3, 4), -1, dtype=torch.int32), torch.zeros(3, dtype=torch.int32), torch.zeros(3, dtype=torch.int32)
    stats = torch.zeros(2, dtype=torch.int64)
    mtp_ops.accept(targets, head_next, None, draft, sampled, seq, out, n_out, arow, stats)
    assert n_out.tolist() == [4, 2, 1] and seq.tolist() == [14, 22, 31]
    assert out.tolist() == [[5, 6, 7, 8], [5, 6, -1, -1], [4, -1, -1, -1]]
    assert sampled.tolist() == [8, 6, 4] and draft[:, 0].tolist() == [103, 105, 108]
    assert stats.tolist() == [9, 4]


def test_scheduler_consumes_multi_token_cycles():
    cfg, eng = _engine(2, max_batch=2)
    sched = ContinuousBatchScheduler(eng)
    done = {}
    for i, n in enumerate((7, 12)):
        p = torch.randint(0, cfg.vocab_size, (n,), generator=torch.Generator().manual_seed(40 + i)).tolist()
        r = Request(prompt=p, params=SamplingParams(max_tokens=9))
        r.on_event = (lambda ev, i=i: done.__setitem__(i, ev) if ev.kind == "completed" else None)
        sched.submit(r)
    sched.run_until_idle()
    assert len(done) == 2 and all(ev.metrics["completion_tokens"] == 9 for ev in done.values())
    assert eng.cache.allocator.free_pages == eng.cache.allocator.num_pages - 1 or eng.free_tokens() > 0


def test_parked_decode_keeps_the_head_primed():
    """A plain step with keep_head leaves draft 1 exactly where a fresh teacher-forced priming over the same context
    puts it: the head's KV rows have no holes after parking."""
    cfg, eng = _engine(2, max_batch=2)
    prompt = torch.randint(0, cfg.vocab_size, (11,), generator=torch.Generator().manual_seed(1))
    eng.active.fill_(0)
    eng.active[0] = 1
    toks = [eng.prefill(0, prompt)]
    agree = 0
    for step in range(5):
        eng.decode_step(1, False, False, keep_head=True)
        eng.row_len[0] += 1
        toks.append(int(eng.sampled[0]))
        _, fresh = _engine(2, max_batch=2)
        ctx = torch.cat([prompt, torch.tensor(toks[:-1], dtype=prompt.dtype)])
        assert fresh.prefill(0, ctx) == toks[-1]  # the main model agrees on the next token
        agree += int(fresh.draft[0, 0]) == int(eng.draft[0, 0])
    assert agree >= 4  # decode and prefill sum in different orders; a near-tie may flip once


def test_adaptive_engine_is_lossless_and_parks_when_cycles_lose():
    from mfq_b200.engine.mtp_policy import ParkingController
    cfg = LlamaConfig.tiny()
    w = LlamaWeights.random_init(cfg, "cpu", seed=5, std=0.05, mtp=True)
    plain_eng = LLMEngine(LlamaModel(cfg, w), max_batch=2, max_seq_len=128, device="cpu")
    adaptive = LLMEngine(LlamaModel(cfg, w), max_batch=2, max_seq_len=128, device="cpu", mtp_draft_tokens=2, mtp_adaptive=True)
    assert isinstance(adaptive.mtp_controller, ParkingController)
    adaptive.mtp_controller = ParkingController(probe=2, park_after=2, reprobe_every=3)
    prompt = list(range(7, 30))
    want = [plain_eng.prefill(0, prompt)]
    plain_eng.grow(0, 128)
    for _ in range(40):
        want.append(plain_eng.decode([0])[0])
    got, modes = [adaptive.prefill(0, prompt)], []
    adaptive.grow(0, 128)
    while len(got) < 36:
        before = dict(adaptive.mtp_controller.calls)
        out = adaptive.decode([0])[0]
        modes.append("mtp" if adaptive.mtp_controller.calls["mtp"] > before["mtp"] else "plain")
        got.extend(out)
    assert "plain" in modes and "mtp" in modes
    assert _agree(want[: len(got)][:32], got[:32]) >= 0.75
    # the decision logic on its own: cycles that lose get parked, a winning re-probe resumes them
    c = ParkingController(probe=2, park_after=3, reprobe_every=4, exit_margin=1.05)
    seen = []
    for i in range(40):
        m = c.mode()
        seen.append(m)
        if m == "mtp":
            c.observe("mtp", tokens=4 if i >= 25 else 1, rows=1, ms=2.0)   # poor acceptance at first, good later
        else:
            c.observe("plain", tokens=1, rows=1, ms=1.0)
    assert seen[:4] == ["mtp", "mtp", "plain", "plain"]
    first_park = next(i for i in range(4, 40) if seen[i] == "plain")
    assert first_park <= 8 and seen[first_park : first_park + 4] == ["plain"] * 4  # parked, then a re-probe
    assert "mtp" in seen[first_park + 4 : first_park + 7]
    assert not c.parked and seen[-3:] == ["mtp"] * 3  # 2 tokens/ms beats 1 token/ms: resumed


def test_dynamic_depth_is_lossless_and_visits_every_depth():
    """Per-cycle depth choice: cycles at 3, 2 and 1 drafts interleave (the controller measures each depth first) and the
    confirmed tokens stay those of plain greedy decoding."""
    cfg, eng = _engine(3, mtp_dynamic_depth=True)
    assert eng.depth_controller is not None
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=torch.Generator().manual_seed(n)) for n in (9, 14)]
    plain = eng.generate(prompts, 14).tokens
    for r in range(2):
        eng.release(r)
    for r, p in enumerate(prompts):
        eng.prefill(r, p)
        eng.grow(r, int(p.numel()) + 40)
    got = {0: [int(eng.sampled[0])], 1: [int(eng.sampled[1])]}
    depths = []
    while min(len(v) for v in got.values()) < 14:
        out = eng.decode([0, 1])
        depths.append(eng.last_depth)
        for r, toks in out.items():
            assert 1 <= len(toks) <= eng.last_depth + 1
            got[r] += toks
    assert set(depths[:6]) == {1, 2, 3}  # every depth gets measured (the next depth is chosen before a cycle is timed)
    assert min(_agree(plain[r].tolist(), got[r][:14]) for r in range(2)) >= 0.75
    st = eng.depth_controller.state()
    assert all(ms is not None for ms in st["cycle_ms"][1:])


def test_stochastic_verification_follows_the_target_distribution():
    """Speculative sampling with the draft head's deterministic proposal: whatever the draft token is, the emitted token
    is distributed as the (temperature / top-k processed) target distribution."""
    cfg, eng = _engine(2, max_batch=1)
    eng.set_sampling(0, SamplingParams(max_tokens=8, temperature=0.8, top_k=5, seed=123))
    v = cfg.vocab_size
    logits = torch.full((3, v), -9.0)
    logits[:, :6] = torch.tensor([2.0, 1.5, 1.0, 0.5, 0.0, -0.5])  # the sixth falls to top-k
    p = torch.softmax(logits[0, :5] / 0.8, -1)
    for draft_tok in (0, 3, 5):  # a likely, an unlikely and an impossible draft
        counts = torch.zeros(v)
        kept = 0
        n = 3000
        for trial in range(n):
            eng.seq_lens[0] = 10 + 3 * trial  # the draw counter: a fresh random number per trial and position
            out = eng._verify_targets(logits, torch.tensor([[draft_tok, 1]], dtype=torch.int32), 1, 3)
            counts[int(out[0])] += 1
            kept += int(out[0]) == draft_tok
        freq = counts[:5] / n
        assert counts[5:].sum() == 0
        assert float((freq - p).abs().max()) < 0.03, (draft_tok, freq.tolist(), p.tolist())
        if draft_tok == 5:
            assert kept == 0
        else:
            assert abs(kept / n - float(p[draft_tok])) < 0.03  # a draft is kept exactly as often as the target would emit it


def test_stochastic_rows_decode_through_mtp_cycles():
    def run():
        cfg, eng = _engine(2, max_batch=2)
        sched = ContinuousBatchScheduler(eng)
        got = {}
        for i, n in enumerate((7, 12)):
            p = torch.randint(0, cfg.vocab_size, (n,), generator=torch.Generator().manual_seed(n)).tolist()
            r = Request(prompt=p, params=SamplingParams(max_tokens=10, temperature=0.9, top_p=0.9, seed=7 + i))
            toks = got.setdefault(i, [])
            def on_event(ev, toks=toks):
                if ev.kind == "token":
                    toks.append(ev.token if hasattr(ev, "token") else ev.data)
                elif ev.kind == "completed":
                    toks.append(("done", ev.metrics["completion_tokens"]))
            r.on_event = on_event
            sched.submit(r)
        sched.run_until_idle()
        return eng, got
    eng, got = run()
    assert all(v[-1] == ("done", 10) for v in got.values())
    st = eng.mtp_stats()
    assert st["cycles"] > 0 and st["drafted"] > 0  # the sampled rows went through draft/verify cycles, not plain steps
    _, again = run()
    assert again == got  # the same seeds replay the same tokens
