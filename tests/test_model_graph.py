"""model_graph.json: built from config + tensor names, embedded in checkpoints, validated when parsed."""

import json

import pytest

from mfq_b200.formats import model_graph as mg


def test_build_and_parse():
    names = [f"model.block.{i}.attention.query.weight" for i in range(3)] + ["model.token_embedding.weight",
             "predictor.block.0.attention.query.weight", "predictor.eh_proj.weight"]
    g = mg.build_graph({"num_layers": 3, "num_experts": 8}, names)
    assert g["graph"] == {"kind": "causal_lm", "backbone": "moe_decoder"}
    assert g["topology"] == {"text_layers": 3, "vision_layers": 0, "predictor_layers": 1}
    assert g["capabilities"] == ["text", "speculative_prediction"] and g["optional_components"]["predictor"]
    assert g["canonical_naming"] == {"namespace": "mfq.tensor", "version": 1, "component_roots": ["model", "predictor"]}
    parsed = mg.parse_graph(mg.to_bytes(g))
    assert parsed.backbone == "moe_decoder" and parsed.predictor_layers == 1 and parsed.has("speculative_prediction")
    assert parsed.unsupported() == []
    vis = mg.parse_graph(mg.build_graph({"num_layers": 1}, names + ["vision.block.0.attn.weight"]))
    assert vis.unsupported() == ["vision"] and vis.vision_layers == 1
    assert mg.backbone_of({"full_attention_interval": 4}) == "hybrid_gdn_moe" and mg.backbone_of({}) == "dense_decoder"


@pytest.mark.parametrize("patch", [{"schema_version": 2}, {"graph": {"kind": "encoder"}},
                                   {"canonical_naming": {"namespace": "other", "component_roots": ["model"]}},
                                   {"canonical_naming": {"namespace": "mfq.tensor", "component_roots": ["vision"]}}])
def test_invalid_graphs_are_rejected(patch):
    g = mg.build_graph({"num_layers": 1}, ["model.block.0.x"])
    g.update(patch)
    with pytest.raises(ValueError):
        mg.parse_graph(json.dumps(g))


def test_checkpoints_carry_the_graph(tmp_path, capsys):
    from mfq_b200 import formats as F
    from mfq_b200.cli import main
    out = tmp_path / "m.mfq"
    assert main(["quantize", "synthetic:tiny-moe", str(out), "--bits", "4"]) == 0
    with F.open_mfq(out) as store:
        g = mg.parse_graph(store.assets()["model_graph.json"])
    assert g.backbone == "moe_decoder" and g.text_layers == 2
    capsys.readouterr()
    assert main(["inspect", str(out)]) == 0
    assert json.loads(capsys.readouterr().out)["graph"]["capabilities"] == ["text"]
