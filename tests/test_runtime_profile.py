"""Sampling profiles: typed validation, merging, registry lookup by fuzzy identity, sidecar files, what `mfq quantize`
embeds, and the server putting a checkpoint's defaults under a request."""

import json

import pytest

from mfq_b200.formats import runtime_profile as rp


def test_validation_is_typed_and_ranged():
    p = rp.make_profile({"temperature": 1, "top_k": 20.0, "enable_mtp": True}, "test", tts={"token2wav_steps": 10})
    assert p["chat"] == {"temperature": 1.0, "top_k": 20, "enable_mtp": True} and isinstance(p["chat"]["temperature"], float)
    assert p["tts"] == {"token2wav_steps": 10} and p["provenance"] == {"source": "test"}
    for bad in ({"temperature": -0.1}, {"top_p": 1.5}, {"top_k": 2.5}, {"enable_mtp": 1}, {"max_tokens": 0}, {"temperature": True},
                {"temperature": float("nan")}, {"nucleus": 0.9}):
        with pytest.raises(ValueError):
            rp.make_profile(bad, "test")
    with pytest.raises(ValueError):
        rp.validate({"schema": rp.SCHEMA, "version": 2, "chat": {}})
    with pytest.raises(ValueError):
        rp.validate({"schema": rp.SCHEMA, "version": 1, "chat": {}, "vision": {}})
    with pytest.raises(ValueError):
        rp.make_profile(None, "t", duplex={"decode_mode": 3})


def test_merge_registry_and_generation_config():
    a = rp.make_profile({"temperature": 0.6, "top_p": 0.9}, "a")
    b = rp.make_profile({"temperature": 0.2}, "b", duplex={"decode_mode": "sampling"})
    m = rp.merge_profiles(a, None, b)
    assert m["chat"] == {"temperature": 0.2, "top_p": 0.9} and m["duplex"] == {"decode_mode": "sampling"} and m["provenance"]["source"] == "b"
    assert rp.merge_profiles(None, None) is None
    assert rp.registry_profile("Qwen3NextForCausalLM")["provenance"]["source"] == "architecture-registry:qwen3_next"
    assert rp.registry_profile("models/DeepSeek-V3-0324")["chat"]["mtp_max_draft_tokens"] == 1
    assert rp.registry_profile("LlamaForCausalLM")["chat"]["top_p"] == 0.9 and rp.registry_profile("mamba") is None
    g = rp.from_generation_config(json.dumps({"max_new_tokens": 512, "temperature": 0.7, "top_k": None, "presence_penalty": 0.5}))
    assert g["chat"] == {"max_tokens": 512, "temperature": 0.7, "presence_penalty": 0.5}
    assert rp.from_generation_config('{"do_sample": false, "temperature": 0.9}')["chat"] == {"temperature": 0.0}
    assert rp.from_generation_config("{}") is None


def test_sidecars_and_resolution_order(tmp_path):
    shard = tmp_path / "model-00001-of-00003.mfq"
    assert rp.sidecar_paths(shard) == (tmp_path / "model.runtime.json", tmp_path / "model-00001-of-00003.mfq.runtime.json")
    single = tmp_path / "tiny.mfq"
    assert rp.sidecar_paths(single) == (tmp_path / "tiny.runtime.json", tmp_path / "tiny.mfq.runtime.json")
    assert rp.load_sidecar(shard) is None
    (tmp_path / "model.runtime.json").write_text(json.dumps(rp.make_profile({"temperature": 0.3, "top_k": 40}, "family")))
    (tmp_path / "model-00001-of-00003.mfq.runtime.json").write_text(json.dumps(rp.make_profile({"temperature": 0.1}, "exact")))
    side = rp.load_sidecar(shard)
    assert side["chat"] == {"temperature": 0.1, "top_k": 40} and side["provenance"]["source"] == "exact"
    embedded = {rp.HEADER_KEY: rp.make_profile({"temperature": 0.8, "top_p": 0.7}, "embedded")}
    gen = {"hf/generation_config.json": b'{"temperature": 0.5, "repetition_penalty": 1.1}'}
    r = rp.resolve(embedded, gen, "llama", shard)
    assert r["source"] == "sidecar" and r["chat"]["temperature"] == 0.1 and r["chat"]["top_k"] == 40      # sidecar
    assert r["chat"]["top_p"] == 0.7 and r["chat"]["repetition_penalty"] == 1.1 and r["chat"]["max_tokens"] == 256  # embedded, gen, builtin
    assert rp.resolve(embedded, gen, "llama")["source"] == "embedded" and rp.resolve(None, gen, "llama")["source"] == "hf-generation-config"
    assert rp.resolve(None, None, "llama")["source"] == "architecture-registry:llama" and rp.resolve()["source"] == "builtin"
    d = rp.checkpoint_defaults({"header_extra": embedded, "assets": gen, "path": str(shard), "architecture": "llama"})
    assert d == {"temperature": 0.1, "repetition_penalty": 1.1, "top_p": 0.7, "top_k": 40}               # nothing from registry / builtin
    (tmp_path / "tiny.runtime.json").write_text('{"schema": "other"}')
    with pytest.raises(ValueError):
        rp.load_sidecar(single)


def test_quantize_embeds_and_server_applies(tmp_path, capsys):
    from fastapi.testclient import TestClient

    from mfq_b200 import formats as F
    from mfq_b200.checkpoint import load_engine
    from mfq_b200.cli import main
    from mfq_b200.server import create_app
    from mfq_b200.server.service import ModelService
    explicit = tmp_path / "profile.json"
    explicit.write_text(json.dumps(rp.make_profile({"max_tokens": 3, "temperature": 0.0}, "operator")))
    out = tmp_path / "tiny.mfq"
    assert main(["quantize", "synthetic:tiny-moe", str(out), "--format", "nint8", "--runtime-profile", str(explicit)]) == 0
    with F.open_mfq(out) as store:
        emb = store.header.extra[rp.HEADER_KEY]
    assert emb["chat"] == {"max_tokens": 3, "temperature": 0.0} and emb["provenance"]["source"] == "operator"
    # re-quantizing the .mfq inherits the profile; without any source of defaults nothing is embedded
    again, bare = tmp_path / "again.mfq", tmp_path / "bare.mfq"
    assert main(["quantize", str(out), str(again), "--format", "nint8"]) == 0
    assert main(["quantize", "synthetic:tiny-moe", str(bare), "--format", "nint8"]) == 0
    with F.open_mfq(again) as a, F.open_mfq(bare) as b:
        assert a.header.extra[rp.HEADER_KEY]["chat"]["max_tokens"] == 3 and rp.HEADER_KEY not in (b.header.extra or {})
    engine, tok, _cfg = load_engine(out, "cpu", max_batch=2, max_seq_len=64)
    assert engine.checkpoint_meta["header_extra"][rp.HEADER_KEY]["chat"]["max_tokens"] == 3
    service = ModelService()
    service.add_model("tiny", engine, tok)
    ask = lambda c, **kw: c.post("/v1/chat/completions", json={"model": "tiny", "messages": [{"role": "user", "content": "hello"}], **kw}).json()
    with TestClient(create_app(service)) as client:
        prof = client.get("/api/v1/runtime/sampling-profile").json()
        assert prof["source"] == "embedded" and prof["chat"]["max_tokens"] == 3
        assert ask(client)["usage"]["completion_tokens"] <= 3                                  # the checkpoint's default
        long = ask(client, max_tokens=6)["usage"]["completion_tokens"]                         # the request wins
        (tmp_path / "tiny.mfq.runtime.json").write_text(json.dumps(rp.make_profile({"max_tokens": 1}, "sidecar")))
        service.models["tiny"].meta.pop("profile_defaults")
        assert ask(client)["usage"]["completion_tokens"] == 1
        assert client.get("/api/v1/runtime/sampling-profile").json()["source"] == "sidecar"
        assert service.models["tiny"].meta["profile_defaults"] == {"max_tokens": 1, "temperature": 0.0}
        assert long >= 1
    service.shutdown()
