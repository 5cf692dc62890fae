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
    for _ in range(20):
        want.append(plain.decode([0])[0])
    got = [spec.prefill(0, prompt)]
    while len(got) < 18:
        got.extend(spec.decode([0])[0])
    agree = 0
    while agree < 16 and want[agree] == got[agree]:
        agree += 1
    assert agree >= 12  # verify windows and one-token steps sum in different orders; a late near-tie may flip
    assert spec.mtp_stats()["drafted"] > 0
