"""A checkpoint with a predictor.* head: stored, loaded, and used for draft/verify decoding through load_engine."""

import numpy as np
import torch

from mfq_b200 import formats as F
from mfq_b200.architectures import canonical_name
from mfq_b200.checkpoint import load_engine, save_checkpoint
from mfq_b200.cli import _SYNTHETIC
from mfq_b200.models.moe_lm import MoeConfig, init_weights


def test_hf_mtp_names_map_to_the_predictor_component():
    assert canonical_name("mtp.fc.weight") == ("predictor.fusion.weight", None)
    assert canonical_name("mtp.pre_fc_norm_hidden.weight") == ("predictor.hidden_norm.weight", None)
    assert canonical_name("mtp.layers.0.self_attn.q_proj.weight") == ("predictor.block.0.attention.query.weight", None)
    assert canonical_name("mtp.layers.0.mlp.experts.5.down_proj.weight") == ("predictor.block.0.mlp.experts.down.weight", 5)


def test_checkpoint_with_a_head_decodes_by_cycles(tmp_path):
    kw = dict(_SYNTHETIC["tiny-moe-128"])
    tensors = {k: v.numpy().astype(np.float32) for k, v in init_weights(MoeConfig(**kw), seed=2, std=0.05).items()}
    rng = np.random.default_rng(9)
    h = kw["hidden_size"]
    # the head: its own block (a copy of block 1's shapes with fresh values), two input norms and the fusion matrix
    for name, t in list(tensors.items()):
        if name.startswith("model.block.1."):
            fresh = np.ones_like(t) if "norm" in name else (rng.standard_normal(t.shape) * 0.05).astype(np.float32)
            tensors["predictor.block.0." + name[len("model.block.1."):]] = fresh
    tensors["predictor.embedding_norm.weight"] = np.ones(h, dtype=np.float32)
    tensors["predictor.hidden_norm.weight"] = np.ones(h, dtype=np.float32)
    tensors["predictor.fusion.weight"] = (rng.standard_normal((h, 2 * h)) * 0.05).astype(np.float32)
    path = tmp_path / "with_head.mfq"
    save_checkpoint(path, dict(kw, name="tiny-with-head"), {k: F.to_bf16(v) for k, v in tensors.items()})
    plain, _, _ = load_engine(path, "cpu", max_batch=2, max_seq_len=96)
    spec, _, _ = load_engine(path, "cpu", max_batch=2, max_seq_len=96, mtp_draft_tokens=2, mtp_adaptive=True)
    assert plain.mtp_k == 0 and plain.model.w.mtp is not None  # loaded, not used unless asked for
    assert spec.mtp_k == 2 and spec.mtp_controller is not None
    prompt = list(range(9, 31))
    want = [plain.prefill(0, prompt)]
    plain.grow(0, 96)
    for _ in range(20):
        want.append(plain.decode([0])[0])
    got = [spec.prefill(0, prompt)]
    spec.grow(0, 96)
    while len(got) < 18:
        got.extend(spec.decode([0])[0])
    agree = 0
    while agree < 16 and want[agree] == got[agree]:
        agree += 1
    assert agree >= 12  # verify windows and one-token steps sum in different orders; a late near-tie may flip
    assert spec.mtp_stats()["drafted"] > 0


def test_base_mfq_gets_a_head_added_without_requantizing(tmp_path, capsys):
    from mfq_b200.cli import main
    kw = dict(_SYNTHETIC["tiny-moe-128"])
    body = {k: v.numpy().astype(np.float32) for k, v in init_weights(MoeConfig(**kw), seed=2, std=0.05).items()}
    base = tmp_path / "base.mfq"
    assert main(["quantize", "synthetic:tiny-moe-128", str(base), "--format", "nint4", "--seed", "2"]) == 0
    # the source of the head: a full-precision checkpoint that carries predictor.* tensors
    rng = np.random.default_rng(1)
    h = kw["hidden_size"]
    head = {"predictor.block.0." + n[len("model.block.1."):]: (np.ones_like(t) if "norm" in n else (rng.standard_normal(t.shape) * 0.05).astype(np.float32))
            for n, t in body.items() if n.startswith("model.block.1.")}
    head.update({"predictor.embedding_norm.weight": np.ones(h, np.float32), "predictor.hidden_norm.weight": np.ones(h, np.float32),
                 "predictor.fusion.weight": (rng.standard_normal((h, 2 * h)) * 0.05).astype(np.float32)})
    src = tmp_path / "with_head_fp.mfq"
    save_checkpoint(src, dict(kw, name="src"), {k: F.to_bf16(v) for k, v in {**body, **head}.items()})
    out = tmp_path / "base_plus_head.mfq"
    assert main(["quantize", str(src), str(out), "--base-mfq", str(base), "--format", "nint8"]) == 0
    capsys.readouterr()
    with F.open_mfq(base) as b, F.open_mfq(out) as o:
        for name in b:
            if not name.startswith("__mfq_asset__/"):
                assert bytes(o.raw(name)) == bytes(b.raw(name)), name  # carried over byte for byte
        assert "predictor.fusion.weight" in o and "predictor.fusion.weight" not in b
    eng, _, _ = load_engine(out, "cpu", max_batch=1, max_seq_len=64, mtp_draft_tokens=2)
    assert eng.mtp_k == 2
    import pytest
    with pytest.raises(SystemExit, match="no multi-token-prediction head"):
        main(["quantize", str(base), str(tmp_path / "x.mfq"), "--base-mfq", str(base)])
