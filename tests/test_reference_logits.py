"""Reference-logits files: round trip, scoring, and byte compatibility with the reference writer."""

import numpy as np
import pytest

from mfq_b200.evaluation import reference_logits as rl


def _model(seed, vocab=50):
    rng = np.random.default_rng(seed)
    table = rng.standard_normal((vocab, vocab)).astype(np.float32) * 2

    def logits(ids):
        return table[np.asarray(ids)]
    return logits


def test_roundtrip_and_scoring(tmp_path):
    rng = np.random.default_rng(0)
    tokens = rng.integers(0, 50, (3, 16))
    base = _model(1)
    nll = rl.write_reference(tmp_path / "ref.bin", tokens, base)
    ref = rl.read_reference(tmp_path / "ref.bin")
    assert (ref.vocab, ref.start, ref.count) == (50, 9, 7) and ref.tokens.shape == (3, 16)
    lp = ref.logp(1)
    want = base(tokens[1])[8:15]
    want = want - want.max(-1, keepdims=True)
    want = want - np.log(np.exp(want).sum(-1, keepdims=True))
    visible = want > -15.5  # entries more than 16 nats below the maximum are clipped by design
    assert np.abs(lp - want)[visible].max() < 3e-4
    assert abs(nll + ref.target_logp.sum()) < 1e-3
    same = rl.score_against_reference(tmp_path / "ref.bin", base)
    assert same["kld"] < 1e-6 and same["same_top"] == 1.0 and abs(same["ppl"] - same["ppl_reference"]) < 1e-3
    other = rl.score_against_reference(tmp_path / "ref.bin", _model(2))
    assert other["kld"] > 0.5 and other["same_top"] < 0.5 and other["tokens"] == 21


def test_bytes_match_reference_writer(reference_pkg, tmp_path):
    from mfq.evaluation.reference import ReferenceWriter
    rng = np.random.default_rng(3)
    tokens = rng.integers(0, 37, (2, 12))
    model = _model(4, vocab=37)
    rl.write_reference(tmp_path / "mine.bin", tokens, model)
    start, count = rl.scored_span(12)
    with ReferenceWriter(tmp_path / "theirs.bin", tokens, 37) as w:
        for c in range(2):
            w.logits(c, 0, model(tokens[c])[start - 1 : 11])
        w.commit()
    assert (tmp_path / "mine.bin").read_bytes() == (tmp_path / "theirs.bin").read_bytes()
