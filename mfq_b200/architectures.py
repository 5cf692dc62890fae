"""Canonical tensor names and the Hugging Face -> canonical mapping for the supported text families.

Runtime code consumes canonical names only (``model.block.N.attention.query.weight`` ...).  Source naming families:

* ``llama``: Llama / Mistral / Qwen2 / Qwen3 dense, Mixtral and Qwen-MoE experts (per-expert or stacked);
* ``qwen3_next``: the hybrid family (``linear_attn.*`` Gated DeltaNet tensors, also in their fused ``in_proj_qkvz`` /
  ``in_proj_ba`` form, ``model.language_model.`` prefix, ``model.visual.*`` kept under ``vision.*``, ``mtp.*`` head);
* ``deepseek_v3`` / ``glm4_moe``: latent-attention and shared-expert names, sigmoid router bias, and the next-token
  prediction layer these checkpoints append after the last decoder layer (``model.layers.<L>.{enorm,hnorm,eh_proj,
  shared_head.*}``), which becomes the ``predictor.*`` head.

:func:`detect_family` picks the family from ``config.json`` (``model_type`` / ``architectures``); :func:`to_canonical`
renames, stacks per-expert matrices, splits fused tensors and moves the appended prediction layer.  Names match the
reference schema (``mfq/architectures/tensor_schema.py:551-596`` text suffixes, ``:630-722`` hybrid family,
``:1745-1900`` DeepSeek families) so checkpoints are interchangeable.
"""

from __future__ import annotations

import re

import numpy as np

TOP_LEVEL = {
    "model.embed_tokens.weight": "model.token_embedding.weight",
    "model.norm.weight": "model.output_norm.weight",
    "lm_head.weight": "model.output.weight",
    "model.language_model.embed_tokens.weight": "model.token_embedding.weight",
    "model.language_model.norm.weight": "model.output_norm.weight",
}
LAYER_SUFFIX = {
    "input_layernorm.weight": "attention.norm.weight",
    "post_attention_layernorm.weight": "mlp.norm.weight",
    "self_attn.q_proj.weight": "attention.query.weight",
    "self_attn.k_proj.weight": "attention.key.weight",
    "self_attn.v_proj.weight": "attention.value.weight",
    "self_attn.o_proj.weight": "attention.output.weight",
    "self_attn.q_a_proj.weight": "attention.query_a.weight",
    "self_attn.q_a_layernorm.weight": "attention.query_a_norm.weight",
    "self_attn.q_b_proj.weight": "attention.query_b.weight",
    "self_attn.kv_a_proj_with_mqa.weight": "attention.key_value_a.weight",
    "self_attn.kv_a_layernorm.weight": "attention.key_value_a_norm.weight",
    "self_attn.kv_b_proj.weight": "attention.key_value_b.source.weight",
    "self_attn.q_norm.weight": "attention.query_norm.weight",
    "self_attn.k_norm.weight": "attention.key_norm.weight",
    "mlp.gate_proj.weight": "mlp.gate.weight",
    "mlp.up_proj.weight": "mlp.up.weight",
    "mlp.down_proj.weight": "mlp.down.weight",
    "mlp.gate.weight": "mlp.router.weight",
    "mlp.gate.e_score_correction_bias": "mlp.router.bias",
    "block_sparse_moe.gate.weight": "mlp.router.weight",
    "mlp.shared_expert.gate_proj.weight": "mlp.shared_expert.gate.weight",
    "mlp.shared_expert.up_proj.weight": "mlp.shared_expert.up.weight",
    "mlp.shared_expert.down_proj.weight": "mlp.shared_expert.down.weight",
    "mlp.shared_experts.gate_proj.weight": "mlp.shared_expert.gate.weight",
    "mlp.shared_experts.up_proj.weight": "mlp.shared_expert.up.weight",
    "mlp.shared_experts.down_proj.weight": "mlp.shared_expert.down.weight",
    "mlp.shared_expert_gate.weight": "mlp.shared_expert.router.weight",
    "mlp.experts.gate_up_proj": "mlp.experts.gate_up.weight",
    "mlp.experts.down_proj": "mlp.experts.down.weight",
    "mlp.experts.gate_up_proj.weight": "mlp.experts.gate_up.weight",
    "mlp.experts.down_proj.weight": "mlp.experts.down.weight",
    "self_attn.q_proj.bias": "attention.query.bias",
    "self_attn.k_proj.bias": "attention.key.bias",
    "self_attn.v_proj.bias": "attention.value.bias",
    # Gated DeltaNet layers of the hybrid family
    "linear_attn.in_proj_qkv.weight": "linear_attention.qkv.weight",
    "linear_attn.in_proj_z.weight": "linear_attention.gate.weight",
    "linear_attn.in_proj_a.weight": "linear_attention.alpha.weight",
    "linear_attn.in_proj_b.weight": "linear_attention.beta.weight",
    "linear_attn.in_proj_qkvz.weight": "linear_attention.qkvz_fused.weight",  # split by to_canonical
    "linear_attn.in_proj_ba.weight": "linear_attention.ba_fused.weight",      # split by to_canonical
    "linear_attn.conv1d.weight": "linear_attention.conv.weight",
    "linear_attn.conv1d.bias": "linear_attention.conv.bias",
    "linear_attn.dt_bias": "linear_attention.dt_bias",
    "linear_attn.A_log": "linear_attention.a",
    "linear_attn.norm.weight": "linear_attention.norm.weight",
    "linear_attn.out_proj.weight": "linear_attention.output.weight",
}
# the prediction layer DeepSeek-V3 / GLM-4.5 style checkpoints append as decoder layer number ``num_hidden_layers``
NEXTN_SUFFIX = {
    "enorm.weight": "predictor.embedding_norm.weight",
    "hnorm.weight": "predictor.hidden_norm.weight",
    "eh_proj.weight": "predictor.fusion.weight",
    "shared_head.norm.weight": "predictor.output_norm.weight",
    "shared_head.head.weight": "predictor.output.weight",
    "embed_tokens.weight": "predictor.token_embedding.weight",
}
VISION_TOP = {
    "patch_embed.proj.weight": "patch_embedding.weight", "patch_embed.proj.bias": "patch_embedding.bias",
    "pos_embed.weight": "position_embedding.weight", "merger.norm.weight": "merger.norm.weight",
    "merger.norm.bias": "merger.norm.bias", "merger.linear_fc1.weight": "merger.mlp.up.weight",
    "merger.linear_fc1.bias": "merger.mlp.up.bias", "merger.linear_fc2.weight": "merger.mlp.down.weight",
    "merger.linear_fc2.bias": "merger.mlp.down.bias",
}
VISION_BLOCK = {
    "norm1.weight": "norm1.weight", "norm1.bias": "norm1.bias", "attn.qkv.weight": "attention.qkv.weight",
    "attn.qkv.bias": "attention.qkv.bias", "attn.proj.weight": "attention.output.weight",
    "attn.proj.bias": "attention.output.bias", "norm2.weight": "norm2.weight", "norm2.bias": "norm2.bias",
    "mlp.linear_fc1.weight": "mlp.up.weight", "mlp.linear_fc1.bias": "mlp.up.bias",
    "mlp.linear_fc2.weight": "mlp.down.weight", "mlp.linear_fc2.bias": "mlp.down.bias",
}
FAMILY_OF_MODEL_TYPE = {
    "llama": "llama", "mistral": "llama", "qwen2": "llama", "qwen3": "llama", "mixtral": "llama", "qwen2_moe": "llama",
    "qwen3_moe": "llama", "qwen3_next": "qwen3_next", "qwen3_5": "qwen3_next", "qwen3_5_moe": "qwen3_next",
    "deepseek_v2": "deepseek_v3", "deepseek_v3": "deepseek_v3", "kimi_k2": "deepseek_v3", "glm4_moe": "glm4_moe",
    "glm4": "llama",
}


def detect_family(hf_config: dict | None, names=()) -> str:
    """Source naming family of a checkpoint: from ``model_type`` (or the text sub-config's), else from its tensor names."""
    cfg = hf_config or {}
    for c in (cfg, cfg.get("text_config") or {}):
        fam = FAMILY_OF_MODEL_TYPE.get(str(c.get("model_type", "")).lower())
        if fam:
            return fam
    for n in names:
        if ".linear_attn." in n or n.startswith("model.language_model."):
            return "qwen3_next"
        if ".kv_a_proj_with_mqa." in n:
            return "deepseek_v3"
    return "llama"
_EXPERT_RE = re.compile(r"^(?:mlp|block_sparse_moe)\.experts\.(\d+)\.(gate_proj|up_proj|down_proj|w1|w2|w3)\.weight$")
_EXPERT_PROJ = {"gate_proj": "gate", "w1": "gate", "up_proj": "up", "w3": "up", "down_proj": "down", "w2": "down"}
_LAYER_RE = re.compile(r"^model\.(?:language_model\.)?layers\.(\d+)\.(.+)$")
_VISION_BLOCK_RE = re.compile(r"^model\.visual\.blocks\.(\d+)\.(.+)$")
# multi-token-prediction head as Qwen3-Next style checkpoints name it
PREDICTOR_TOP = {
    "mtp.fc.weight": "predictor.fusion.weight",
    "mtp.pre_fc_norm_embedding.weight": "predictor.embedding_norm.weight",
    "mtp.pre_fc_norm_hidden.weight": "predictor.hidden_norm.weight",
    "mtp.norm.weight": "predictor.output_norm.weight",
}
_MTP_LAYER_RE = re.compile(r"^mtp\.layers\.(\d+)\.(.+)$")


def canonical_name(hf_name: str, nextn_layer: int | None = None) -> tuple[str, int | None] | None:
    """``hf_name`` -> (canonical name, expert index or None); None for tensors the runtime does not use.
    ``nextn_layer``: index of the appended prediction layer (= ``num_hidden_layers``) of the families that have one."""
    if hf_name in TOP_LEVEL:
        return TOP_LEVEL[hf_name], None
    if hf_name in PREDICTOR_TOP:
        return PREDICTOR_TOP[hf_name], None
    if hf_name.startswith("model.visual."):
        rest = hf_name[len("model.visual."):]
        if rest in VISION_TOP:
            return "vision." + VISION_TOP[rest], None
        v = _VISION_BLOCK_RE.match(hf_name)
        if v and v[2] in VISION_BLOCK:
            return f"vision.block.{int(v[1])}.{VISION_BLOCK[v[2]]}", None
        return None
    m, root = _LAYER_RE.match(hf_name), "model"
    if not m:
        m, root = _MTP_LAYER_RE.match(hf_name), "predictor"
    if not m:
        return None
    layer, rest = int(m[1]), m[2]
    if root == "model" and nextn_layer is not None and layer >= nextn_layer:
        if rest in NEXTN_SUFFIX:
            return NEXTN_SUFFIX[rest], None
        root, layer = "predictor", layer - nextn_layer
    if rest in LAYER_SUFFIX:
        return f"{root}.block.{layer}.{LAYER_SUFFIX[rest]}", None
    e = _EXPERT_RE.match(rest)
    if e:
        return f"{root}.block.{layer}.mlp.experts.{_EXPERT_PROJ[e[2]]}.weight", int(e[1])
    return None


def split_fused_linear_attention(out: dict[str, np.ndarray], k_heads: int, v_heads: int, head_dim: int) -> None:
    """The hybrid family's fused projections, in place: ``in_proj_qkvz`` holds, per KEY head, the rows
    ``[q (d) | k (d) | v (r d) | z (r d)]`` with ``r = v_heads / k_heads``; ``in_proj_ba`` holds ``[b (r) | a (r)]`` per
    key head.  They become the separate ``qkv`` (rows q | k | v, heads contiguous), ``gate``, ``beta`` and ``alpha``
    matrices of the canonical schema."""
    r, d = v_heads // k_heads, head_dim
    for name in [n for n in out if n.endswith("linear_attention.qkvz_fused.weight")]:
        w = out.pop(name)
        per = w.reshape(k_heads, 2 * d + 2 * r * d, w.shape[-1])
        q, k = per[:, :d], per[:, d : 2 * d]
        v, z = per[:, 2 * d : 2 * d + r * d], per[:, 2 * d + r * d :]
        base = name[: -len("qkvz_fused.weight")]
        out[base + "qkv.weight"] = np.concatenate([q.reshape(-1, w.shape[-1]), k.reshape(-1, w.shape[-1]), v.reshape(-1, w.shape[-1])])
        out[base + "gate.weight"] = np.ascontiguousarray(z.reshape(-1, w.shape[-1]))
    for name in [n for n in out if n.endswith("linear_attention.ba_fused.weight")]:
        w = out.pop(name)
        per = w.reshape(k_heads, 2 * r, w.shape[-1])
        base = name[: -len("ba_fused.weight")]
        out[base + "beta.weight"] = np.ascontiguousarray(per[:, :r].reshape(-1, w.shape[-1]))
        out[base + "alpha.weight"] = np.ascontiguousarray(per[:, r:].reshape(-1, w.shape[-1]))


def to_canonical(hf_tensors: dict[str, np.ndarray], hf_config: dict | None = None) -> dict[str, np.ndarray]:
    """Rename a Hugging Face state dict; per-expert matrices are stacked into ``[experts, out, in]`` tensors, a fused
    ``gate_up`` expert tensor is split into ``gate`` and ``up``, fused linear-attention projections are split, and the
    prediction layer appended after the decoder stack moves under ``predictor.*``.  ``hf_config`` (the checkpoint's
    ``config.json``) selects the family and supplies the geometry those steps need."""
    family = detect_family(hf_config, hf_tensors)
    text = dict(hf_config or {})
    text.update(text.get("text_config") or {})
    nextn = None
    if family in ("deepseek_v3", "glm4_moe") and text.get("num_hidden_layers") and text.get("num_nextn_predict_layers", 0):
        nextn = int(text["num_hidden_layers"])
    out: dict[str, np.ndarray] = {}
    experts: dict[str, dict[int, np.ndarray]] = {}
    for name, t in hf_tensors.items():
        mapped = canonical_name(name, nextn)
        if mapped is None:
            continue
        cname, e = mapped
        if e is None:
            out[cname] = t
        else:
            experts.setdefault(cname, {})[e] = t
    for cname, parts in experts.items():
        out[cname] = np.stack([parts[i] for i in range(len(parts))])
    for cname in [n for n in out if n.endswith("mlp.experts.gate_up.weight")]:
        fused = out.pop(cname)
        half = fused.shape[1] // 2
        out[cname.replace("gate_up", "gate")] = fused[:, :half]
        out[cname.replace("gate_up", "up")] = fused[:, half:]
    if any(n.endswith("_fused.weight") for n in out):
        kh, vh = text.get("linear_num_key_heads"), text.get("linear_num_value_heads")
        hd = text.get("linear_key_head_dim") or text.get("linear_value_head_dim")
        if not (kh and vh and hd):
            raise ValueError("fused linear-attention projections need linear_num_key_heads / linear_num_value_heads / "
                             "linear_key_head_dim from config.json")
        split_fused_linear_attention(out, int(kh), int(vh), int(hd))
    if family == "qwen3_next" and text.get("attn_output_gate", True) and text.get("num_attention_heads"):
        # the hybrid family's q_proj emits, per head, [query (d) | output gate (d)]: split into the two canonical matrices
        heads = int(text["num_attention_heads"])
        d = int(text.get("head_dim") or text["hidden_size"] // heads)
        for cname in [n for n in out if n.endswith(".attention.query.weight") and out[n].shape[0] == 2 * heads * d]:
            per = out[cname].reshape(heads, 2 * d, -1)
            out[cname] = np.ascontiguousarray(per[:, :d].reshape(heads * d, -1))
            out[cname.replace("query.weight", "gate.weight")] = np.ascontiguousarray(per[:, d:].reshape(heads * d, -1))
    if "model.output.weight" not in out and "model.token_embedding.weight" in out:
        out["model.output.weight"] = out["model.token_embedding.weight"]  # tied embeddings
    return out


def config_from_hf(hf: dict) -> dict:
    """``config.json`` of a Hugging Face model -> the keyword arguments of ``MoeDecoderConfig`` (and of its hybrid and
    latent-attention extensions); a multimodal wrapper's ``text_config`` is looked through."""
    if hf.get("text_config"):
        hf = {**hf, **hf["text_config"]}
    heads = hf.get("num_attention_heads", 32)
    cfg = {
        "vocab_size": hf["vocab_size"], "hidden_size": hf["hidden_size"], "num_layers": hf["num_hidden_layers"],
        "num_heads": heads, "num_kv_heads": hf.get("num_key_value_heads", heads),
        "head_dim": hf.get("head_dim") or hf["hidden_size"] // heads, "intermediate_size": hf.get("intermediate_size", 0),
        "rope_theta": float(hf.get("rope_theta", 1e4)), "rms_eps": float(hf.get("rms_norm_eps", 1e-5)),
        "name": hf.get("_name_or_path") or hf.get("model_type", "model"),
    }
    from .models.rope_scaling import YarnScaling
    yarn = YarnScaling.from_hf(hf)
    if yarn is not None:
        cfg["rope_scaling"] = yarn.to_dict()
        cfg["max_position"] = int(hf.get("max_position_embeddings") or yarn.max_position())
    if hf.get("linear_num_value_heads"):  # hybrid family: Gated DeltaNet layers between full-attention layers
        cfg.update(linear_k_heads=int(hf.get("linear_num_key_heads", 16)), linear_v_heads=int(hf["linear_num_value_heads"]),
                   linear_head_dim=int(hf.get("linear_key_head_dim", 128)),
                   full_attention_interval=int(hf.get("full_attention_interval", 4)),
                   partial_rotary=float(hf.get("partial_rotary_factor", 0.25)),
                   attn_output_gate=bool(hf.get("attn_output_gate", True)))
    if hf.get("kv_lora_rank"):  # latent attention (DeepSeek-V2/V3 style)
        cfg.update(q_lora_rank=int(hf.get("q_lora_rank") or 0), kv_lora_rank=int(hf["kv_lora_rank"]),
                   qk_nope_head_dim=int(hf.get("qk_nope_head_dim", 128)), qk_rope_head_dim=int(hf.get("qk_rope_head_dim", 64)),
                   v_head_dim=int(hf.get("v_head_dim", 128)))
    experts = hf.get("num_experts") or hf.get("num_local_experts") or hf.get("n_routed_experts") or 0
    if experts:
        cfg.update(num_experts=experts, top_k=hf.get("num_experts_per_tok", 2),
                   moe_intermediate=hf.get("moe_intermediate_size") or hf.get("intermediate_size"),
                   shared_intermediate=hf.get("shared_expert_intermediate_size", 0) or
                   hf.get("n_shared_experts", 0) * (hf.get("moe_intermediate_size") or 0),
                   router="sigmoid" if hf.get("scoring_func") == "sigmoid" else "softmax",
                   norm_topk=bool(hf.get("norm_topk_prob", True)), routed_scale=float(hf.get("routed_scaling_factor", 1.0)),
                   n_group=hf.get("n_group", 1) or 1, topk_group=hf.get("topk_group", 1) or 1,
                   first_dense_layers=hf.get("first_k_dense_replace", 0))
    return cfg
