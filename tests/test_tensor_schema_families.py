"""Source naming families of the canonical tensor schema: hybrid (fused linear-attention projections, fused query|gate,
multimodal prefixes, mtp head), DeepSeek / GLM style appended prediction layer, detection from config and names."""

import numpy as np

from mfq_b200.architectures import canonical_name, config_from_hf, detect_family, to_canonical
from mfq_b200.models.hybrid import HybridConfig, init_hybrid_weights


def _hybrid_as_hf(cfg, w, prefix="model.language_model."):
    """The tiny hybrid model's canonical tensors renamed (and fused) the way the hybrid family's checkpoints store them."""
    kh, vh, d = cfg.linear_k_heads, cfg.linear_v_heads, cfg.linear_head_dim
    r = vh // kh
    hf = {prefix + "embed_tokens.weight": w["model.token_embedding.weight"], prefix + "norm.weight": w["model.output_norm.weight"],
          "lm_head.weight": w["model.output.weight"]}
    plain = {"attention.norm.weight": "input_layernorm.weight", "mlp.norm.weight": "post_attention_layernorm.weight",
             "mlp.router.weight": "mlp.gate.weight", "mlp.shared_expert.gate.weight": "mlp.shared_expert.gate_proj.weight",
             "mlp.shared_expert.up.weight": "mlp.shared_expert.up_proj.weight", "mlp.shared_expert.down.weight": "mlp.shared_expert.down_proj.weight",
             "attention.key.weight": "self_attn.k_proj.weight", "attention.value.weight": "self_attn.v_proj.weight",
             "attention.output.weight": "self_attn.o_proj.weight", "attention.query_norm.weight": "self_attn.q_norm.weight",
             "attention.key_norm.weight": "self_attn.k_norm.weight", "linear_attention.conv.weight": "linear_attn.conv1d.weight",
             "linear_attention.a": "linear_attn.A_log", "linear_attention.dt_bias": "linear_attn.dt_bias",
             "linear_attention.norm.weight": "linear_attn.norm.weight", "linear_attention.output.weight": "linear_attn.out_proj.weight"}
    for layer in range(cfg.num_layers):
        c, h = f"model.block.{layer}.", f"{prefix}layers.{layer}."
        for cn, hn in plain.items():
            if c + cn in w:
                hf[h + hn] = w[c + cn]
        for proj, hn in (("gate", "gate_proj"), ("up", "up_proj"), ("down", "down_proj")):
            for e, m in enumerate(w[c + f"mlp.experts.{proj}.weight"]):
                hf[h + f"mlp.experts.{e}.{hn}.weight"] = m
        if c + "linear_attention.qkv.weight" in w:
            qkv, z = w[c + "linear_attention.qkv.weight"], w[c + "linear_attention.gate.weight"]
            cols = qkv.shape[1]
            q, k, v = qkv[: kh * d].reshape(kh, d, cols), qkv[kh * d : 2 * kh * d].reshape(kh, d, cols), qkv[2 * kh * d :].reshape(kh, r * d, cols)
            hf[h + "linear_attn.in_proj_qkvz.weight"] = np.concatenate([q, k, v, z.reshape(kh, r * d, cols)], axis=1).reshape(-1, cols)
            a, b = w[c + "linear_attention.alpha.weight"].reshape(kh, r, cols), w[c + "linear_attention.beta.weight"].reshape(kh, r, cols)
            hf[h + "linear_attn.in_proj_ba.weight"] = np.concatenate([b, a], axis=1).reshape(-1, cols)
        else:
            heads, hd = cfg.num_heads, cfg.head_dim
            q, g = w[c + "attention.query.weight"].reshape(heads, hd, -1), w[c + "attention.gate.weight"].reshape(heads, hd, -1)
            hf[h + "self_attn.q_proj.weight"] = np.concatenate([q, g], axis=1).reshape(2 * heads * hd, -1)
    return hf


def test_hybrid_family_round_trip_through_source_names():
    cfg = HybridConfig.tiny()
    w = {k: np.asarray(v.float().numpy()) for k, v in init_hybrid_weights(cfg, seed=2, std=0.05).items()}
    hf_cfg = {"model_type": "qwen3_5_moe", "text_config": {
        "model_type": "qwen3_5_moe_text", "num_hidden_layers": cfg.num_layers, "num_attention_heads": cfg.num_heads,
        "head_dim": cfg.head_dim, "hidden_size": cfg.hidden_size, "linear_num_key_heads": cfg.linear_k_heads,
        "linear_num_value_heads": cfg.linear_v_heads, "linear_key_head_dim": cfg.linear_head_dim, "attn_output_gate": True}}
    hf = _hybrid_as_hf(cfg, w)
    hf["model.visual.patch_embed.proj.weight"] = np.zeros((4, 3, 2, 2), np.float32)
    hf["model.visual.blocks.1.attn.qkv.weight"] = np.zeros((6, 2), np.float32)
    hf["mtp.fc.weight"] = np.zeros((4, 8), np.float32)
    hf["mtp.layers.0.self_attn.k_proj.weight"] = np.zeros((4, 4), np.float32)
    assert detect_family(hf_cfg) == "qwen3_next" and detect_family(None, hf) == "qwen3_next"
    back = to_canonical(hf, hf_cfg)
    for name, t in w.items():
        assert np.array_equal(back[name], t), name
    assert "vision.patch_embedding.weight" in back and "vision.block.1.attention.qkv.weight" in back
    assert "predictor.fusion.weight" in back and "predictor.block.0.attention.key.weight" in back
    assert not [n for n in back if "_fused" in n]


def test_hybrid_config_keys_reach_the_model_config():
    kw = config_from_hf({"model_type": "qwen3_next", "vocab_size": 100, "hidden_size": 256, "num_hidden_layers": 4,
                         "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 128, "linear_num_key_heads": 2,
                         "linear_num_value_heads": 4, "linear_key_head_dim": 128, "full_attention_interval": 2,
                         "partial_rotary_factor": 0.25, "num_experts": 8, "num_experts_per_tok": 2, "moe_intermediate_size": 128,
                         "shared_expert_intermediate_size": 128})
    cfg = HybridConfig(**kw)
    assert cfg.linear_v_heads == 4 and cfg.full_attention_interval == 2 and cfg.is_linear(0) and not cfg.is_linear(1)


def test_appended_prediction_layer_becomes_the_predictor():
    hf_cfg = {"model_type": "deepseek_v3", "num_hidden_layers": 2, "num_nextn_predict_layers": 1}
    z = np.zeros((2, 2), np.float32)
    hf = {"model.embed_tokens.weight": z, "model.norm.weight": z[0], "lm_head.weight": z,
          "model.layers.0.self_attn.kv_a_proj_with_mqa.weight": z, "model.layers.1.mlp.gate.e_score_correction_bias": z[0],
          "model.layers.1.mlp.experts.0.gate_proj.weight": z, "model.layers.1.mlp.experts.1.gate_proj.weight": z + 1,
          "model.layers.2.enorm.weight": z[0], "model.layers.2.hnorm.weight": z[0], "model.layers.2.eh_proj.weight": z,
          "model.layers.2.shared_head.norm.weight": z[0], "model.layers.2.shared_head.head.weight": z,
          "model.layers.2.embed_tokens.weight": z, "model.layers.2.self_attn.q_a_proj.weight": z,
          "model.layers.2.mlp.shared_experts.up_proj.weight": z, "model.layers.2.input_layernorm.weight": z[0]}
    assert detect_family(hf_cfg) == "deepseek_v3" and detect_family({"model_type": "glm4_moe"}) == "glm4_moe"
    assert detect_family(None, hf) == "deepseek_v3"
    out = to_canonical(hf, hf_cfg)
    assert {"predictor.embedding_norm.weight", "predictor.hidden_norm.weight", "predictor.fusion.weight",
            "predictor.output_norm.weight", "predictor.output.weight", "predictor.token_embedding.weight",
            "predictor.block.0.attention.query_a.weight", "predictor.block.0.mlp.shared_expert.up.weight",
            "predictor.block.0.attention.norm.weight"} <= set(out)
    assert out["model.block.1.mlp.experts.gate.weight"].shape == (2, 2, 2) and out["model.block.1.mlp.experts.gate.weight"][1, 0, 0] == 1
    assert "model.block.1.mlp.router.bias" in out and "model.block.2.attention.query_a.weight" not in out
    # without the config the appended layer cannot be told from a decoder layer: it stays a block
    assert canonical_name("model.layers.2.self_attn.q_a_proj.weight") == ("model.block.2.attention.query_a.weight", None)
