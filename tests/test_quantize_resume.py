"""Resumable quantization: parked per-tensor blobs are reused only when source, plan and payload still match."""

import json

import numpy as np
import pytest

from mfq_b200 import formats as F
from mfq_b200.checkpoint import quantize_tensors
from mfq_b200.cli import main
from mfq_b200.quantize.resume import ResumeStore


def _tensors(seed=0):
    rng = np.random.default_rng(seed)
    return {"model.layers.0.self_attn.q_proj.weight": rng.standard_normal((64, 128)).astype(np.float32),
            "model.layers.0.mlp.down_proj.weight": rng.standard_normal((128, 64)).astype(np.float32),
            "model.norm.weight": np.ones(128, dtype=np.float32)}


def test_interrupted_run_is_picked_up(tmp_path, monkeypatch):
    t = _tensors()
    full = quantize_tensors(t, dense="nint4")
    store = ResumeStore(tmp_path / "x.tmp")
    import mfq_b200.quantize as Q
    real, calls = Q.quantize_matrix, []

    def dying(a, profile, **kw):
        calls.append(a.shape)
        if len(calls) == 2:
            raise KeyboardInterrupt
        return real(a, profile, **kw)

    monkeypatch.setattr(Q, "quantize_matrix", dying)
    with pytest.raises(KeyboardInterrupt):
        quantize_tensors(t, dense="nint4", resume=store)
    assert store.written == ["model.layers.0.self_attn.q_proj.weight"]
    monkeypatch.setattr(Q, "quantize_matrix", real)
    again = ResumeStore(tmp_path / "x.tmp", resume=True)
    out = quantize_tensors(t, dense="nint4", resume=again)
    assert again.reused == ["model.layers.0.self_attn.q_proj.weight"] and len(again.written) == 2
    for k in t:
        assert F.pack_tensor(out[k]) == F.pack_tensor(full[k])
    again.finish()
    assert not (tmp_path / "x.tmp").exists()


def test_changed_plan_source_or_damaged_blob_requantizes(tmp_path):
    t = _tensors()
    name = "model.layers.0.self_attn.q_proj.weight"
    s = ResumeStore(tmp_path / "r", keep=True)
    quantize_tensors(t, dense="nint4", resume=s)
    s.finish()
    assert (tmp_path / "r").exists()  # keep
    s2 = ResumeStore(tmp_path / "r", resume=True, keep=True)
    quantize_tensors(t, dense="nint8", resume=s2)  # another plan
    assert name not in s2.reused
    s3 = ResumeStore(tmp_path / "r", resume=True, keep=True)
    t2 = dict(t)
    t2[name] = t[name] + 1.0  # another source
    quantize_tensors(t2, dense="nint8", resume=s3)
    assert name not in s3.reused and "model.layers.0.mlp.down_proj.weight" in s3.reused
    blob = s3._path(name)
    blob.write_bytes(blob.read_bytes()[:-7])  # cut short
    s4 = ResumeStore(tmp_path / "r", resume=True, keep=True)
    assert s4.get(name, s4.key(name, t2[name], "whatever")) is None
    quantize_tensors(t2, dense="nint8", resume=s4)
    assert name in s4.written
    assert not ResumeStore(tmp_path / "r").dir.joinpath(blob.name).exists()  # without resume the directory starts empty


def test_cli_flags(tmp_path, capsys):
    out = tmp_path / "m.mfq"
    assert main(["quantize", "synthetic:tiny-moe", str(out), "--format", "nint4", "--keep-temp"]) == 0
    first = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert first["resumed_tensors"] == 0 and (tmp_path / "m.mfq.tmp").is_dir()
    ref = out.read_bytes()
    assert main(["quantize", "synthetic:tiny-moe", str(out), "--format", "nint4", "--overwrite", "--resume"]) == 0
    second = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert second["resumed_tensors"] > 10 and out.read_bytes() == ref and not (tmp_path / "m.mfq.tmp").exists()
    assert main(["quantize", "synthetic:tiny-moe", str(out), "--format", "nint4", "--resume-completed"]) == 0
    assert json.loads(capsys.readouterr().out.strip().splitlines()[-1])["already_complete"] is True
