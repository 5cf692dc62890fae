"""Structured output end to end on the CPU engine: a random model constrained to JSON emits a valid object."""

import json

import pytest
import torch

from mfq_b200.engine.llm_engine import LLMEngine
from mfq_b200.engine.scheduler import ContinuousBatchScheduler, Request, SamplingParams
from mfq_b200.models.llama import LlamaConfig, LlamaModel, LlamaWeights
from mfq_b200.server.tokenizer import ByteTokenizer


def _engine():
    cfg = LlamaConfig.tiny()
    eng = LLMEngine(LlamaModel(cfg, LlamaWeights.random_init(cfg, "cpu", seed=7)), max_batch=4, max_seq_len=160, device="cpu")
    tok = ByteTokenizer(cfg.vocab_size)
    eng.set_token_bytes(lambda: tok.token_bytes(cfg.vocab_size), tok.stop_ids)
    return eng, tok


def _run(sched, reqs, steps=400):
    for r in reqs:
        sched.submit(r)
    for _ in range(steps):
        if not sched.step() and sched.idle:
            break


@pytest.mark.parametrize("temperature", [0.0, 0.9])
def test_constrained_rows_emit_json_and_free_rows_are_untouched(temperature):
    eng, tok = _engine()
    sched = ContinuousBatchScheduler(eng, max_queue=8)
    prompt = tok.encode("Reply in JSON.")
    free_alone = Request(list(prompt), SamplingParams(max_tokens=24, stop_token_ids=tok.stop_ids))
    _run(sched, [free_alone])
    fmt = SamplingParams(max_tokens=120, temperature=temperature, seed=3, stop_token_ids=tok.stop_ids,
                         response_format={"type": "json_object"})
    a = Request(list(prompt), fmt)
    b = Request(tok.encode("Another one, in JSON please."), fmt)
    free = Request(list(prompt), SamplingParams(max_tokens=24, stop_token_ids=tok.stop_ids))
    _run(sched, [a, free, b])
    assert free.generated == free_alone.generated  # a neighbour's constraint does not leak into this row
    for r in (a, b):
        text = tok.decode([t for t in r.generated if t not in tok.stop_ids])
        assert text.lstrip().startswith("{")
        if r.finish_reason == "stop":  # ended by itself: the document is complete
            assert isinstance(json.loads(text), dict), text
        else:  # ran into max_tokens: still a valid prefix
            from mfq_b200 import native
            s = native.JsonState(eng._constraint_vocab, need_object=True)
            assert s.feed(text.encode())
    assert not eng.row_constraint  # released with the rows


def test_a_complete_document_can_only_be_followed_by_the_end():
    eng, tok = _engine()
    fmt = SamplingParams(max_tokens=8, stop_token_ids=tok.stop_ids, response_format={"type": "json_object"})
    prompt, doc = tok.encode("JSON:"), tok.encode('{"a": [1, true]}')
    t1 = eng.prefill(0, prompt + doc, fmt, generated=len(doc))
    allowed_ws = {b + 3 for b in b" \n\t\r"}
    assert t1 in allowed_ws or t1 == tok.eos_id
    if t1 != tok.eos_id:
        assert eng.decode([0])[0] == tok.eos_id  # one trailing whitespace byte at most
    c = eng.row_constraint[0]
    assert c.finished
    eng.release(0)
    # an unfinished document: the end-of-sequence token is masked out
    t2 = eng.prefill(0, prompt + tok.encode('{"a"'), fmt, generated=4)
    assert t2 in allowed_ws or t2 == ord(":") + 3


def test_replay_after_retraction_restores_the_grammar_state():
    eng, tok = _engine()
    fmt = SamplingParams(max_tokens=64, stop_token_ids=tok.stop_ids, response_format={"type": "json_object"})
    prompt = tok.encode("JSON:")
    first = eng.prefill(0, prompt, fmt)
    out = [first]
    for _ in range(5):
        out.append(eng.decode([0])[0])
    nxt = eng.decode([0])[0]
    eng.release(0)
    # the same request re-admitted with its context so far (what the scheduler does after a retraction)
    again = eng.prefill(1, prompt + out, fmt, generated=len(out))
    assert again == nxt
    eng.release(1)


def test_server_parses_response_format():
    from mfq_b200.server.app import _params_from
    assert _params_from({"response_format": {"type": "json_object"}}, ()).response_format == {"type": "json_object"}
    assert _params_from({"response_format": {"type": "text"}}, ()).response_format is None
    assert _params_from({}, ()).response_format is None
    with pytest.raises(ValueError):
        _params_from({"response_format": {"type": "xml"}}, ())


def test_metrics_render_with_a_real_engine():
    """/metrics over an LLMEngine (KV gauges, resident bytes, MTP ratio only once something was drafted)."""
    from mfq_b200.server import ModelService
    eng, tok = _engine()
    service = ModelService()
    try:
        service.add_model("tiny", eng, tok)
        text = service.metrics.render(service)
        assert 'mfq_runtime_kv_bytes{' in text and "mfq_runtime_resident_bytes{" in text and "mfq_runtime_mtp_acceptance_ratio" not in text
        rss = float([l for l in text.splitlines() if l.startswith("mfq_runtime_resident_bytes{")][0].split()[-1])
        assert rss > 50e6
    finally:
        service.shutdown()


def test_logit_bias_bans_and_forces_tokens():
    eng, tok = _engine()
    prompt = tok.encode("abc")
    free = [eng.prefill(0, prompt, SamplingParams(max_tokens=8))]
    for _ in range(5):
        free.append(eng.decode([0])[0])
    eng.release(0)
    banned = {t: -100 for t in set(free)}
    got = [eng.prefill(0, prompt, SamplingParams(max_tokens=8, logit_bias=banned))]
    for _ in range(5):
        got.append(eng.decode([0])[0])
    eng.release(0)
    assert not set(got) & set(free)
    forced = [eng.prefill(0, prompt, SamplingParams(max_tokens=8, logit_bias={77: 100}))]
    forced.append(eng.decode([0])[0])
    assert forced == [77, 77]
    from mfq_b200.server.app import _params_from
    assert _params_from({"logit_bias": {"12": -5, "13": 250}}, ()).logit_bias == {12: -5.0, 13: 250.0}
