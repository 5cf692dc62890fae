"""Recipes (GGUF tensor table / JSON rules), AlphaQ target bits per weight, shard limits."""

import json

import numpy as np
import pytest

from mfq_b200 import formats as F
from mfq_b200.cli import main
from mfq_b200.formats import gguf as G
from mfq_b200.quantize.recipe import load_recipe, parse_size, widths_from_rules


def test_sizes_and_rules():
    assert parse_size("500M") == 500 << 20 and parse_size("4G") == 4 << 30 and parse_size("1.5k") == 1536 and parse_size("77") == 77
    with pytest.raises(ValueError):
        parse_size("big")
    names = ["model.block.0.attention.query.weight", "model.block.0.mlp.down.weight", "model.output.weight"]
    plan = widths_from_rules({"rules": [{"match": r"attention\.", "bits": 6}, {"match": r"output\.weight$", "bits": None}], "default": 3}, names)
    assert plan == {names[0]: 6, names[1]: 3, names[2]: None}
    with pytest.raises(ValueError):
        widths_from_rules({"rules": [{"match": ".", "bits": 9}]}, names)


def test_gguf_tensor_table_as_recipe(tmp_path):
    path = tmp_path / "recipe.gguf"
    z = np.zeros((32, 64), dtype=np.float32)
    G.write_gguf(path, {"general.architecture": "llama"}, {
        "blk.0.attn_q.weight": (z, G.GGML_Q8_0), "blk.0.ffn_down.weight": (z, G.GGML_Q4_0), "output_norm.weight": (np.zeros(64, np.float32), G.GGML_F32),
        "token_embd.weight": (z, G.GGML_F16)})
    names = ["model.block.0.attention.query.weight", "model.block.0.mlp.down.weight", "model.token_embedding.weight", "model.block.1.mlp.down.weight"]
    assert load_recipe(path, names) == {names[0]: 8, names[1]: 4, names[2]: None}


def test_cli_recipe_target_bpw_and_shard_limits(tmp_path, capsys):
    recipe = tmp_path / "r.json"
    recipe.write_text(json.dumps({"rules": [{"match": r"attention\.(query|key)\.", "bits": 8}, {"match": r"attention\.value", "bits": None}], "default": 3}))
    out = tmp_path / "m.mfq"
    assert main(["quantize", "synthetic:tiny-moe", str(out), "--recipe", str(recipe), "--backend", "cpu", "--split-max-tensors", "7"]) == 0
    info = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert info["shards"] >= 3
    with F.open_mfq(info["output"]) as store:
        q, v, o = (store[f"model.block.0.attention.{n}.weight"] for n in ("query", "value", "output"))
        assert store.dtype("model.block.0.attention.value.weight") in ("BF16", "bf16")
        assert max(q.row_q_bits) == 8 if hasattr(q, "row_q_bits") and q.row_q_bits is not None else True
    lo, hi = tmp_path / "lo.mfq", tmp_path / "hi.mfq"
    assert main(["quantize", "synthetic:tiny-moe", str(lo), "--target-bpw", "3.0"]) == 0
    a = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert main(["quantize", "synthetic:tiny-moe", str(hi), "--target-bpw", "6.0", "--split-max-size", "200k"]) == 0
    b = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert b["bytes"] > a["bytes"] * 1.2 and b["shards"] > 1 and a["shards"] == 1
