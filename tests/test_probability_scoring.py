"""Probability scoring: `LLMEngine.score` against the reference language model, additivity over split continuations,
the control route, and the serving thread owning the engine while it runs."""

import json

import numpy as np
import torch

from mfq_b200.checkpoint import load_engine
from mfq_b200.cli import main


def _engine(tmp_path):
    out = tmp_path / "tiny.mfq"
    assert main(["quantize", "synthetic:tiny-moe", str(out), "--full-precision"]) == 0
    return out, load_engine(out, "cpu", max_batch=2, max_seq_len=96)


def test_engine_scores_match_a_plain_forward(tmp_path, capsys):
    from mfq_b200 import formats as F
    from mfq_b200.models.moe_lm import MoeConfig, MoeLM, dequantize_checkpoint
    path, (engine, tok, cfg) = _engine(tmp_path)
    ids = torch.randint(0, cfg.vocab_size, (40,), generator=torch.Generator().manual_seed(1)).tolist()
    got = engine.score(0, ids, 25)
    assert len(got) == 15 and all(x <= 0 for x in got) and 0 not in engine.row_seq       # the scratch row is free again
    with F.open_mfq(path) as store:
        raw = json.loads(store.assets()["model_config.json"])
        tensors = {n: store[n] for n in store if not n.startswith("__mfq_asset__/")}
    lm = MoeLM(MoeConfig(**{k: v for k, v in raw.items() if k in MoeConfig.__dataclass_fields__}), dequantize_checkpoint(tensors))
    logp = torch.log_softmax(lm.forward(torch.tensor(ids)).float(), -1)
    want = [float(logp[p - 1, ids[p]]) for p in range(25, 40)]
    assert np.allclose(got, want, atol=0.08), (got[:3], want[:3])                         # FP8 activations vs fp32
    # chunked: the same numbers when the span crosses prefill chunks
    engine.prefill_chunk = 16
    assert np.allclose(engine.score(1, ids, 25), got, atol=1e-4)
    # a continuation scored in two parts adds up
    a = engine.score(0, ids[:30], 25)
    b = engine.score(0, ids, 30)
    assert np.allclose(a + b, got, atol=1e-4)
    for bad in ((ids, 0), (ids, 40), (ids * 3, 5)):
        try:
            engine.score(0, *bad)
            raise AssertionError("accepted")
        except ValueError:
            pass


def test_route_scores_continuations(tmp_path, capsys):
    from fastapi.testclient import TestClient

    from mfq_b200.server import create_app
    from mfq_b200.server.service import ModelService
    _path, (engine, tok, _cfg) = _engine(tmp_path)
    service = ModelService()
    service.add_model("tiny", engine, tok)
    with TestClient(create_app(service)) as c:
        r = c.post("/api/v1/evaluations/probabilities", json={"prompt": "The sky is", "continuations": [" blue", " green tea"]}).json()
        assert r["log_base"] == "e" and r["tokenization"] == "raw-no-special-tokens" and r["prompt_tokens"] == len(tok.encode("The sky is"))
        assert [len(s["token_ids"]) for s in r["scores"]] == [len(tok.encode(" blue")), len(tok.encode(" green tea"))]
        for s in r["scores"]:
            assert len(s["token_logprobs"]) == len(s["token_ids"]) and abs(sum(s["token_logprobs"]) - s["log_likelihood"]) < 1e-6
            assert all(x <= 0 for x in s["token_logprobs"])
        first = c.post("/api/v1/evaluations/probabilities", json={"prompt": "The sky is", "continuations": [" blue"], "mode": "next_token"}).json()
        assert len(first["scores"][0]["token_ids"]) == 1
        assert abs(first["scores"][0]["token_logprobs"][0] - r["scores"][0]["token_logprobs"][0]) < 1e-6
        # a generation afterwards still works: the scratch row was handed back
        g = c.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "hi"}], "max_tokens": 3}).json()
        assert g["usage"]["completion_tokens"] >= 1
        assert c.post("/api/v1/evaluations/probabilities", json={"prompt": "x", "continuations": []}).status_code == 400
        assert c.post("/api/v1/evaluations/probabilities", json={"prompt": "x", "continuations": ["y"], "mode": "beam"}).status_code == 400
        assert c.post("/api/v1/evaluations/probabilities", json={"model": "nope", "prompt": "x", "continuations": ["y"]}).status_code == 404
    service.shutdown()


def test_scope_of_the_route():
    from mfq_b200.server.auth import required_scope
    assert required_scope("POST", "/api/v1/evaluations/probabilities") == "inference"
    assert required_scope("POST", "/api/v1/jobs") == "admin"
