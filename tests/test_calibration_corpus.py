"""Calibration corpora (text and generated traces) and the activation / Fisher statistics collected over them."""

import json

import numpy as np
import pytest
import torch

from mfq_b200 import cli
from mfq_b200.calibration import dataset, statistics
from mfq_b200.server.tokenizer import ByteTokenizer


def _write_jsonl(path, rows):
    path.write_text("\n".join(json.dumps(r) for r in rows))


def _sources(tmp_path):
    rng = np.random.default_rng(0)
    words = ["alpha", "beta", "gamma", "delta", "tensor", "kernel", "cache", "token", "norm", "rope"]
    a = [{"text": " ".join(rng.choice(words, 30))} for _ in range(60)]
    b = [{"messages": [{"role": "user", "content": " ".join(rng.choice(words, 8))},
                       {"role": "assistant", "content": " ".join(rng.choice(words, 20))}]} for _ in range(60)]
    _write_jsonl(tmp_path / "a.jsonl", a)
    _write_jsonl(tmp_path / "b.jsonl", b)
    return a, b


def test_pack_stream_never_leaves_a_single_token():
    for n in range(2, 40):
        for sl in (2, 3, 8):
            chunks = dataset.pack_stream(list(range(n)), sl)
            assert sum(c.size for c in chunks) == n and min(c.size for c in chunks) >= 2
            assert np.concatenate(chunks).tolist() == list(range(n))
            assert max(c.size for c in chunks) <= max(sl, 3)


def test_text_corpus_quotas_splits_and_reload(tmp_path):
    a, b = _sources(tmp_path)
    tok = ByteTokenizer()
    corpus = dataset.build_text_corpus(tok, tmp_path / "corpus", {"plain": a, "chat": b}, train_tokens=4000, validation_tokens=600,
                                       sequence_length=128, seed=3, domain_weights={"plain": 3, "chat": 1})
    m = corpus.manifest
    assert m["format"] == dataset.FORMAT and m["actual_tokens"] == {"train": 4000, "validation": 600}
    assert corpus.token_count("train") == 4000 and corpus.token_count("validation") == 600
    # domain shares: 3:1 in both splits
    sizes = np.diff(corpus.offsets)
    for split, total in (("train", 4000), ("validation", 600)):
        sel = corpus.split_ids == dataset.SPLITS[split]
        plain = sizes[sel & (corpus.domain_ids == m["domains"].index("plain"))].sum()
        assert plain == total * 3 // 4
    assert max(sizes) <= 128 and min(sizes) >= 2
    # the two splits use different records
    for d in m["domains"]:
        assert m["record_sets"]["train"][d]["sha256"] != m["record_sets"]["validation"][d]["sha256"]
    again = dataset.load_corpus(tmp_path / "corpus")
    assert np.array_equal(again.tokens, corpus.tokens) and again.manifest["token_sha256"] == m["token_sha256"]
    # same seed, same corpus; another seed, another order
    same = dataset.build_text_corpus(tok, tmp_path / "c2", {"plain": a, "chat": b}, train_tokens=4000, validation_tokens=600,
                                     sequence_length=128, seed=3, domain_weights={"plain": 3, "chat": 1})
    other = dataset.build_text_corpus(tok, tmp_path / "c3", {"plain": a, "chat": b}, train_tokens=4000, validation_tokens=600,
                                      sequence_length=128, seed=4, domain_weights={"plain": 3, "chat": 1})
    assert same.manifest["token_sha256"] == m["token_sha256"] != other.manifest["token_sha256"]
    with pytest.raises(ValueError):
        dataset.build_text_corpus(tok, tmp_path / "c4", {"plain": a[:2]}, train_tokens=10 ** 6, validation_tokens=10, sequence_length=64)
    # a tampered token file is refused
    t = np.load(tmp_path / "c2" / "tokens.npy")
    t[0] += 1
    np.save(tmp_path / "c2" / "tokens.npy", t)
    with pytest.raises(ValueError):
        dataset.load_corpus(tmp_path / "c2")


def _traces(n):
    rows = []
    for i in range(n):
        thinking = i % 3 == 0
        rows.append({"model": "Gen-1", "mode": "thinking" if thinking else "nonthinking", "finish_reason": "stop",
                     "messages": [{"role": "user", "content": f"question number {i} about kernels"}],
                     "output": f"answer {i}: use shared memory " * 3, "reasoning": "think " * 5 if thinking else None,
                     "source_dataset": "unit"})
    rows.append({"model": "Other", "mode": "nonthinking", "finish_reason": "stop", "messages": [{"role": "user", "content": "x"}], "output": "y"})
    rows.append({"model": "Gen-1", "mode": "nonthinking", "finish_reason": "length", "messages": [{"role": "user", "content": "x"}], "output": "y"})
    return rows


def test_trace_corpus_scores_only_generated_positions(tmp_path):
    tok = ByteTokenizer()
    corpus = dataset.build_trace_corpus(tok, tmp_path / "traces", _traces(40), train_tokens=3000, validation_tokens=500,
                                        sequence_length=1024, seed=1, expected_generator_model="gen-1")
    m = corpus.manifest
    assert m["format"] == dataset.MASKED_FORMAT and corpus.loss_mask is not None
    assert sum(m["excluded"].values()) >= 1  # the foreign-model / cut-off rows never enter
    for i in range(corpus.chunks):
        toks, mask = corpus.chunk_tokens(i), corpus.chunk_loss_mask(i)
        text = tok.decode(toks.tolist())
        first = int(np.flatnonzero(mask)[0])
        assert mask[0] == 0 and mask[first:].all()  # one scored run at the end: the generated turn
        assert "question number" in tok.decode(toks[:first].tolist()) and "answer" in tok.decode(toks[first:].tolist())
        assert "answer" not in tok.decode(toks[: first - 12].tolist()) or "question" in text
    assert m["scored_tokens"] == int(corpus.loss_mask.sum()) < corpus.tokens.size
    with pytest.raises(ValueError):
        dataset.trace_record({"model": "Gen-1", "mode": "thinking", "finish_reason": "stop", "messages": [{"role": "user", "content": "q"}], "output": "a"})


def test_statistics_collect_save_load(tmp_path):
    from mfq_b200.models.moe_lm import MoeConfig, init_weights
    cfg = MoeConfig(**cli._SYNTHETIC["tiny-moe-128"])
    w = init_weights(cfg, seed=2)
    a, b = _sources(tmp_path)

    class Tok(ByteTokenizer):  # ids inside the tiny vocabulary
        pass
    corpus = dataset.build_text_corpus(Tok(), tmp_path / "corpus", {"plain": a, "chat": b}, train_tokens=1200, validation_tokens=400,
                                       sequence_length=64, seed=0)
    stats = statistics.collect_statistics(cfg, {k: v.numpy() for k, v in w.items()}, corpus, tmp_path / "stats.npz",
                                          train_input_tokens=1200, validation_input_tokens=400, train_fisher_tokens=256,
                                          validation_fisher_tokens=128)
    q = stats.require("model.block.0.attention.query.weight")
    assert q.target.rows == cfg.num_heads * cfg.head_dim and q.target.columns == cfg.hidden_size
    assert q.train_input_count == 1200 and q.validation_input_count == 400
    assert 0 < q.train_fisher_probes <= 256 and q.train_row_fisher.shape == (q.target.rows,)
    assert float(q.train_row_fisher.max()) > 1e-12 and float(q.train_input_second_moment.min()) > 0
    # Fisher of a row = mean of (dL/dy_r)^2 |x|^2: check one layer against a direct autograd computation on one window
    head = stats.require("model.output.weight")
    assert head.target.rows == cfg.vocab_size and float(head.train_row_fisher.sum()) > float(q.train_row_fisher.sum()) * 1e-6
    # experts: inputs and exposure only
    ex = [n for n in stats.entries if "#" in n]
    assert ex and all(stats.entries[n].train_fisher_probes == 0 for n in ex)
    im = stats.as_imatrix()
    assert "model.block.1.mlp.shared_expert.down.weight.in" in im
    again = statistics.load_statistics(tmp_path / "stats.npz")
    assert np.allclose(again.require(q.target.name).train_row_fisher, q.train_row_fisher)
    assert again.metadata["corpus"]["token_sha256"] == corpus.manifest["token_sha256"]
    with pytest.raises(FileExistsError):
        statistics.save_statistics(tmp_path / "stats.npz", stats.entries, {})


def test_row_fisher_matches_direct_gradient():
    """One projection, one window: the hook's row sums equal the squared weight gradient summed along rows when the
    window has a single scored position (then no cross terms between positions exist)."""
    torch.manual_seed(0)
    acc = statistics._Accumulator(fisher=True)
    w = torch.randn(5, 7, requires_grad=True)
    x = torch.randn(1, 7, requires_grad=True)
    y = x @ w.T
    acc.observe("p", x, y)
    loss = (y ** 2).sum()
    loss.backward()
    assert torch.allclose(acc.sum_fisher["p"].float(), (w.grad ** 2).sum(1), rtol=1e-5)
    assert acc.n_fisher["p"] == 1


def test_cli_data_trace_collect(tmp_path, capsys):
    _sources(tmp_path)
    _write_jsonl(tmp_path / "t.jsonl", _traces(30))
    assert cli.main(["calibrate", "data", "--source", f"plain={tmp_path / 'a.jsonl'}", "--source", f"chat={tmp_path / 'b.jsonl'}",
                     "--output", str(tmp_path / "corpus"), "--train-tokens", "1500", "--validation-tokens", "300",
                     "--sequence-length", "64"]) == 0
    ev = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert ev["event"] == "calibration_corpus_ready" and ev["train_tokens"] == 1500
    assert cli.main(["calibrate", "trace-data", "--source-file", str(tmp_path / "t.jsonl"), "--expected-generator-model", "Gen-1",
                     "--output", str(tmp_path / "traces"), "--train-tokens", "1500", "--validation-tokens", "300",
                     "--sequence-length", "512"]) == 0
    ev = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert ev["event"] == "trace_calibration_corpus_ready"
    assert cli.main(["calibrate", "collect", "synthetic:tiny-moe", "--corpus", str(tmp_path / "traces"), "--output",
                     str(tmp_path / "s.npz"), "--imatrix-output", str(tmp_path / "im.npz"), "--train-input-tokens", "600",
                     "--validation-input-tokens", "200", "--train-fisher-tokens", "200", "--validation-fisher-tokens", "100"]) == 0
    ev = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert ev["event"] == "calibration_statistics_ready" and ev["tensors"] > 10
    from mfq_b200.calibration.imatrix import load
    assert any(k.endswith(".in") for k in load(tmp_path / "im.npz"))


def test_imatrix_over_a_corpus(tmp_path, capsys):
    _sources(tmp_path)
    assert cli.main(["calibrate", "data", "--source", str(tmp_path / "a.jsonl"), "--output", str(tmp_path / "corpus"),
                     "--train-tokens", "900", "--validation-tokens", "100", "--sequence-length", "64"]) == 0
    capsys.readouterr()
    assert cli.main(["calibrate", "imatrix", "synthetic:tiny-moe", "--output", str(tmp_path / "im.npz"), "--corpus",
                     str(tmp_path / "corpus"), "--chunks", "6", "--ctx", "64"]) == 0
    ev = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert ev["tokens"] == 6 * 64 and ev["layers"] > 5
    from mfq_b200.calibration.imatrix import load
    im = load(tmp_path / "im.npz")
    assert int(im["model.block.0.attention.query.weight.count"]) == 6 * 64
