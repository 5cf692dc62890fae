"""Canonical tensor names and the Hugging Face -> canonical mapping for the supported text families.

Runtime code consumes canonical names only (``model.block.N.attention.query.weight`` ...); the mapping table below
covers Llama/Mistral/Qwen dense models, Mixtral/Qwen-MoE style experts (per-expert or stacked), DeepSeek shared
experts and the MTP predictor (``predictor.*``).  Names match the reference schema
(``mfq/architectures/tensor_schema.py:551-596``) so checkpoints are interchangeable.
"""

from __future__ import annotations

import re

import numpy as np

TOP_LEVEL = {
    "model.embed_tokens.weight": "model.token_embedding.weight",
    "model.norm.weight": "model.output_norm.weight",
    "lm_head.weight": "model.output.weight",
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
}
_EXPERT_RE = re.compile(r"^(?:mlp|block_sparse_moe)\.experts\.(\d+)\.(gate_proj|up_proj|down_proj|w1|w2|w3)\.weight$")
_EXPERT_PROJ = {"gate_proj": "gate", "w1": "gate", "up_proj": "up", "w3": "up", "down_proj": "down", "w2": "down"}
_LAYER_RE = re.compile(r"^model\.layers\.(\d+)\.(.+)$")
# multi-token-prediction head as Qwen3-Next style checkpoints name it
PREDICTOR_TOP = {
    "mtp.fc.weight": "predictor.fusion.weight",
    "mtp.pre_fc_norm_embedding.weight": "predictor.embedding_norm.weight",
    "mtp.pre_fc_norm_hidden.weight": "predictor.hidden_norm.weight",
    "mtp.norm.weight": "predictor.output_norm.weight",
}
_MTP_LAYER_RE = re.compile(r"^mtp\.layers\.(\d+)\.(.+)$")


def canonical_name(hf_name: str) -> tuple[str, int | None] | None:
    """``hf_name`` -> (canonical name, expert index or None); None for tensors the runtime does not use."""
    if hf_name in TOP_LEVEL:
        return TOP_LEVEL[hf_name], None
    if hf_name in PREDICTOR_TOP:
        return PREDICTOR_TOP[hf_name], None
    m, root = _LAYER_RE.match(hf_name), "model"
    if not m:
        m, root = _MTP_LAYER_RE.match(hf_name), "predictor"
    if not m:
        return None
    layer, rest = int(m[1]), m[2]
    if rest in LAYER_SUFFIX:
        return f"{root}.block.{layer}.{LAYER_SUFFIX[rest]}", None
    e = _EXPERT_RE.match(rest)
    if e:
        return f"{root}.block.{layer}.mlp.experts.{_EXPERT_PROJ[e[2]]}.weight", int(e[1])
    return None


def to_canonical(hf_tensors: dict[str, np.ndarray]) -> dict[str, np.ndarray]:
    """Rename a Hugging Face state dict; per-expert matrices are stacked into ``[experts, out, in]`` tensors and a
    fused ``gate_up`` expert tensor is split into ``gate`` and ``up``."""
    out: dict[str, np.ndarray] = {}
    experts: dict[str, dict[int, np.ndarray]] = {}
    for name, t in hf_tensors.items():
        mapped = canonical_name(name)
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
    if "model.output.weight" not in out and "model.token_embedding.weight" in out:
        out["model.output.weight"] = out["model.token_embedding.weight"]  # tied embeddings
    return out


def config_from_hf(hf: dict) -> dict:
    """``config.json`` of a Hugging Face model -> the keyword arguments of ``MoeDecoderConfig``."""
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
