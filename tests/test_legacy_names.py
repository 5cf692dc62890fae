"""Artifacts that stored Hugging Face tensor paths load through a canonical-name view."""

import json

import numpy as np
import pytest
import torch

from mfq_b200 import formats as F
from mfq_b200.checkpoint import load_engine, save_checkpoint
from mfq_b200.formats.legacy_names import canonical_view
from mfq_b200.models.llama import LlamaConfig


def _dense_tensors(cfg, rng):
    h, d = cfg.hidden_size, cfg.head_dim
    t = {"model.embed_tokens.weight": rng.standard_normal((cfg.vocab_size, h)) * 0.05, "model.norm.weight": np.ones(h),
         "lm_head.weight": rng.standard_normal((cfg.vocab_size, h)) * 0.05}
    for i in range(cfg.num_layers):
        p = f"model.layers.{i}."
        t[p + "input_layernorm.weight"] = np.ones(h)
        t[p + "post_attention_layernorm.weight"] = np.ones(h)
        t[p + "self_attn.q_proj.weight"] = rng.standard_normal((cfg.num_heads * d, h)) * 0.05
        t[p + "self_attn.k_proj.weight"] = rng.standard_normal((cfg.num_kv_heads * d, h)) * 0.05
        t[p + "self_attn.v_proj.weight"] = rng.standard_normal((cfg.num_kv_heads * d, h)) * 0.05
        t[p + "self_attn.o_proj.weight"] = rng.standard_normal((h, cfg.num_heads * d)) * 0.05
        t[p + "mlp.gate_proj.weight"] = rng.standard_normal((cfg.intermediate_size, h)) * 0.05
        t[p + "mlp.up_proj.weight"] = rng.standard_normal((cfg.intermediate_size, h)) * 0.05
        t[p + "mlp.down_proj.weight"] = rng.standard_normal((h, cfg.intermediate_size)) * 0.05
    return {k: v.astype(np.float32) for k, v in t.items()}


def test_old_artifact_loads_like_its_canonical_twin(tmp_path):
    from mfq_b200.architectures import to_canonical
    cfg = LlamaConfig.tiny()
    raw = dict(vocab_size=cfg.vocab_size, hidden_size=cfg.hidden_size, intermediate_size=cfg.intermediate_size, num_layers=cfg.num_layers,
               num_heads=cfg.num_heads, num_kv_heads=cfg.num_kv_heads, head_dim=cfg.head_dim, rope_theta=cfg.rope_theta,
               rms_eps=cfg.rms_eps, num_experts=0)
    hf = _dense_tensors(cfg, np.random.default_rng(0))
    old, new = tmp_path / "old.mfq", tmp_path / "new.mfq"
    save_checkpoint(old, raw, {k: F.to_bf16(v) for k, v in hf.items()})
    save_checkpoint(new, raw, {k: F.to_bf16(v) for k, v in to_canonical(hf).items()})
    with F.open_mfq(old) as store:
        view = canonical_view(store)
        assert "model.block.0.attention.query.weight" in view and "model.token_embedding.weight" in set(view)
        assert view.assets()["model_config.json"]
    with F.open_mfq(new) as store:
        assert canonical_view(store) is store
    ids = torch.arange(4, 30)
    a = load_engine(old, "cpu", max_batch=1, max_seq_len=64)[0].generate([ids], 5).tokens
    b = load_engine(new, "cpu", max_batch=1, max_seq_len=64)[0].generate([ids], 5).tokens
    assert torch.equal(a, b)


def test_per_expert_source_names_are_refused_with_the_fix():
    store = {"model.layers.0.mlp.experts.3.up_proj.weight": object(), "__mfq_asset__/model_config.json": b"{}"}
    with pytest.raises(ValueError, match="mfq quantize"):
        canonical_view(store)
