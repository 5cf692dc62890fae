"""Hugging Face directories: safetensors reader, name mapping, quantizing from one and serving one directly."""

import json
import struct

import numpy as np
import torch

from mfq_b200.architectures import LAYER_SUFFIX, TOP_LEVEL
from mfq_b200.checkpoint import load_engine, read_hf_directory
from mfq_b200.cli import _SYNTHETIC, main
from mfq_b200.models.moe_lm import MoeConfig, init_weights


def _write_safetensors(path, tensors):
    header, blobs, off = {}, [], 0
    for name, a in tensors.items():
        raw = np.ascontiguousarray(a, dtype=np.float32).tobytes()
        header[name] = {"dtype": "F32", "shape": list(a.shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    h = json.dumps(header).encode()
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(h)) + h + b"".join(blobs))


def _hf_directory(tmp_path):
    """A Qwen-MoE style checkpoint directory built from the synthetic tiny model (names mapped back to HF's)."""
    kw = _SYNTHETIC["tiny-moe-128"]
    canon = {k: v.numpy().astype(np.float32) for k, v in init_weights(MoeConfig(**kw), seed=4).items()}
    back_top = {v: k for k, v in TOP_LEVEL.items()}
    back_layer = {}
    for hf, c in LAYER_SUFFIX.items():
        back_layer.setdefault(c, hf)  # first spelling wins (shared_expert before shared_experts)
    hf = {}
    for name, t in canon.items():
        if name in back_top:
            hf[back_top[name]] = t
            continue
        _, _, layer, rest = name.split(".", 3)
        if rest.startswith("mlp.experts."):
            proj = rest.split(".")[2]
            for e in range(t.shape[0]):
                hf[f"model.layers.{layer}.mlp.experts.{e}.{proj}_proj.weight"] = t[e]
        else:
            hf[f"model.layers.{layer}.{back_layer[rest]}"] = t
    d = tmp_path / "hf"
    d.mkdir()
    names = sorted(hf)
    _write_safetensors(d / "model-00001-of-00002.safetensors", {n: hf[n] for n in names[: len(names) // 2]})
    _write_safetensors(d / "model-00002-of-00002.safetensors", {n: hf[n] for n in names[len(names) // 2 :]})
    (d / "config.json").write_text(json.dumps({
        "model_type": "qwen2_moe", "vocab_size": kw["vocab_size"], "hidden_size": kw["hidden_size"],
        "num_hidden_layers": kw["num_layers"], "num_attention_heads": kw["num_heads"], "num_key_value_heads": kw["num_kv_heads"],
        "head_dim": kw["head_dim"], "rope_theta": kw["rope_theta"], "rms_norm_eps": kw["rms_eps"], "num_experts": kw["num_experts"],
        "num_experts_per_tok": kw["top_k"], "moe_intermediate_size": kw["moe_intermediate"],
        "shared_expert_intermediate_size": kw["shared_intermediate"], "norm_topk_prob": True}))
    return d, canon


def test_reader_maps_names_and_stacks_experts(tmp_path):
    d, canon = _hf_directory(tmp_path)
    cfg, tensors, assets = read_hf_directory(d)
    assert cfg["num_experts"] == 8 and cfg["top_k"] == 2 and cfg["head_dim"] == 128 and assets == {}
    assert set(tensors) == set(canon)
    for k in canon:
        assert tensors[k].shape == canon[k].shape and np.array_equal(tensors[k], canon[k]), k


def test_quantize_from_and_serve_a_directory(tmp_path, capsys):
    d, _ = _hf_directory(tmp_path)
    out = tmp_path / "m.mfq"
    assert main(["quantize", str(d), str(out), "--full-precision"]) == 0
    capsys.readouterr()
    ids = torch.arange(5, 29)
    from_file, _, cfg_a = load_engine(out, "cpu", max_batch=1, max_seq_len=64)
    direct, _, cfg_b = load_engine(d, "cpu", max_batch=1, max_seq_len=64)
    assert cfg_a.num_experts == cfg_b.num_experts == 8
    a = from_file.generate([ids], 6).tokens
    b = direct.generate([ids], 6).tokens
    assert a.shape == (1, 6) and torch.equal(a, b)
