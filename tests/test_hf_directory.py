"""Hugging Face directories: safetensors reader, name mapping, quantizing from one and serving one directly."""

import json
import struct

import numpy as np
import pytest
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


def test_prequantized_sources_fold_to_float():
    """Block-scaled FP8, tensor- and channel-scaled FP8 and MXFP4 block/scale pairs become plain float matrices."""
    from mfq_b200.checkpoint import fold_source_quantization
    from mfq_b200.formats.mx import dequantize_mx
    from mfq_b200.quantize.mxfp4 import quantize_mxfp4
    rng = np.random.default_rng(0)
    codes = rng.normal(size=(200, 300)).astype(np.float32)            # stands for decoded E4M3 values
    grid = rng.uniform(0.5, 2.0, size=(2, 3)).astype(np.float32)
    per_row = rng.uniform(0.5, 2.0, size=(200, 1)).astype(np.float32)
    src = quantize_mxfp4((rng.normal(size=(6, 64)) * 0.1).astype(np.float32))
    blocks = np.asarray(src.values).reshape(6, 2, 16)
    t = fold_source_quantization({
        "a.weight": codes, "a.weight_scale_inv": grid,
        "b.weight": codes, "b.weight_scale": np.array([0.25], dtype=np.float32), "b.input_scale": np.array([3.0], dtype=np.float32),
        "c.weight": codes, "c.weight_scale": per_row,
        "experts.down_proj_blocks": np.stack([blocks, blocks]), "experts.down_proj_scales": np.stack([src.scales, src.scales]),
        "norm.weight": np.ones(4, dtype=np.float32)}, {"quantization_config": {"weight_block_size": [128, 128]}})
    assert set(t) == {"a.weight", "b.weight", "c.weight", "experts.down_proj", "norm.weight"}
    assert np.allclose(t["a.weight"][130, 260], codes[130, 260] * grid[1, 2]) and np.allclose(t["a.weight"][5, 5], codes[5, 5] * grid[0, 0])
    assert np.allclose(t["b.weight"], codes * 0.25) and np.allclose(t["c.weight"], codes * per_row)
    assert t["experts.down_proj"].shape == (2, 6, 64) and np.array_equal(t["experts.down_proj"][1], dequantize_mx(src))
    with pytest.raises(ValueError):
        fold_source_quantization({"a.weight": codes, "a.weight_scale_inv": grid[:1]})


def test_block_fp8_directory_reads_like_its_float_twin(tmp_path):
    """A directory whose projections are stored as E4M3 + ``weight_scale_inv`` grids reads to (nearly) the float model."""
    from mfq_b200.formats.mx import e4m3_to_float, float_to_e4m3
    d, canon = _hf_directory(tmp_path)
    shard = d / "model-00001-of-00002.safetensors"
    from mfq_b200.checkpoint import read_safetensors
    tensors = read_safetensors(shard)
    header, blobs, off = {}, [], 0
    changed = 0
    for name, a in tensors.items():
        if name.endswith("proj.weight") and a.ndim == 2 and a.shape[0] % 128 == 0 and a.shape[1] % 128 == 0:
            r, c = a.shape[0] // 128, a.shape[1] // 128
            amax = np.abs(a.reshape(r, 128, c, 128)).max((1, 3))
            scale = np.maximum(amax, 1e-12) / 448.0
            q = float_to_e4m3(a / np.repeat(np.repeat(scale, 128, 0), 128, 1))
            for nm, arr, dt in ((name, q, "F8_E4M3"), (name + "_scale_inv", scale.astype(np.float32), "F32")):
                raw = np.ascontiguousarray(arr).tobytes()
                header[nm] = {"dtype": dt, "shape": list(arr.shape), "data_offsets": [off, off + len(raw)]}
                blobs.append(raw)
                off += len(raw)
            changed += 1
        else:
            raw = np.ascontiguousarray(a, dtype=np.float32).tobytes()
            header[name] = {"dtype": "F32", "shape": list(a.shape), "data_offsets": [off, off + len(raw)]}
            blobs.append(raw)
            off += len(raw)
    assert changed > 0
    h = json.dumps(header).encode()
    shard.write_bytes(struct.pack("<Q", len(h)) + h + b"".join(blobs))
    cfg = json.loads((d / "config.json").read_text())
    cfg["quantization_config"] = {"quant_method": "fp8", "weight_block_size": [128, 128]}
    (d / "config.json").write_text(json.dumps(cfg))
    _, got, _ = read_hf_directory(d)
    assert set(got) == set(canon)
    worst = max(float(np.abs(got[k] - canon[k]).max() / max(np.abs(canon[k]).max(), 1e-12)) for k in canon)
    assert 0 < worst < 0.07   # E4M3 rounding only: 3 mantissa bits
