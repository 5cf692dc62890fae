"""Presets, AlphaQ statistics/allocation, imatrix collection and the expert-wise MILP solver."""

import numpy as np
import pytest
import torch

from mfq_b200.calibration import alphaq, ew_solver, imatrix
from mfq_b200.quantize import presets
from mfq_b200.quantize.nint import quantize_nint
from mfq_b200.formats import nint


def test_preset_role_rules():
    topo = presets.Topology(layers=32, heads=32, kv_heads=8)
    v = "model.block.{}.attention.value.weight"
    down = "model.block.{}.mlp.down.weight"
    assert presets.select_bits("S4-M", v.format(0), topo) == 6 and presets.select_bits("S4-M", v.format(5), topo) == 4
    assert presets.select_bits("s4_m", down.format(31), topo) == 6
    assert presets.select_bits("S2-M", v.format(3), topo) == 4  # GQA >= 4 protects the shared value heads
    assert presets.select_bits("S2-M", down.format(3), topo) == 3
    assert presets.select_bits("S3-M", down.format(0), topo) == 5 and presets.select_bits("S3-M", down.format(4), topo) == 3
    assert presets.select_bits("S4-S", "model.output.weight", topo) == 6 and presets.select_bits("S8", "model.output.weight", topo) == 8
    assert presets.select_bits("S3-S", "model.block.1.mlp.shared_expert.up.weight", topo) == 8
    assert presets.select_bits("S3-S", "model.block.1.linear_attention.alpha.weight", topo) == 8
    assert presets.select_bits("S5-S", "model.block.9.attention.query.weight", topo) == 5
    with pytest.raises(ValueError):
        presets.normalize_preset("S7")
    shapes = {"model.block.0.attention.value.weight": (1024, 4096), "model.block.0.attention.norm.weight": (4096,),
              "model.block.0.mlp.router.weight": (8, 4096), "model.block.0.mlp.experts.down.weight": (8, 4096, 512),
              "model.block.0.linear_attention.conv.weight": (8192, 1, 4)}
    p = presets.plan("S4-M", shapes, topo)
    assert p["model.block.0.attention.norm.weight"] is None and p["model.block.0.mlp.router.weight"] is None
    assert p["model.block.0.linear_attention.conv.weight"] is None and p["model.block.0.mlp.experts.down.weight"] == 4
    assert [presets.more_bits(i, 32) for i in range(8)] == [True, True, True, True, False, False, True, False]


def test_alphaq_statistics_and_allocation():
    rng = np.random.default_rng(0)
    gauss = rng.standard_normal((256, 256)).astype(np.float32) * 0.02
    heavy = (rng.standard_t(2.0, (256, 256)) * 0.02).astype(np.float32)  # heavy tails -> smaller alpha
    sg, sh = alphaq.weight_statistics(gauss), alphaq.weight_statistics(heavy)
    assert sh.alpha < sg.alpha and sh.variance > sg.variance
    assert alphaq.weight_statistics(np.ones((64, 64), np.float32)).variance == 0.0
    assert abs(alphaq.hill_alpha(np.array([5.0])) - 1.0) < 1e-12
    stats = {"gauss": sg, "heavy": sh, "small": alphaq.weight_statistics(gauss[:100, :90] * 0.1)}
    imp = alphaq.importance(stats)
    assert imp["heavy"] == max(imp.values()) and imp["small"] == min(imp.values())
    sizes = {k: s.size for k, s in stats.items()}
    cands = {"NINT2": 2.6, "NINT3": 3.5, "NINT4": 4.5, "NINT6": 6.5}
    total = sum(sizes.values())
    choice = alphaq.allocate(imp, sizes, cands, budget_bits=4.0 * total)
    used = sum(sizes[k] * cands[c] for k, c in choice.items())
    assert used <= 4.0 * total and cands[choice["heavy"]] >= cands[choice["gauss"]] >= cands[choice["small"]]
    with pytest.raises(ValueError):
        alphaq.allocate(imp, sizes, cands, budget_bits=1.0 * total)


def test_imatrix_weights_reduce_weighted_error(tmp_path):
    g = torch.Generator().manual_seed(0)
    w = torch.randn((64, 128), generator=g) * 0.05
    scale = torch.ones(128)
    scale[:16] = 12.0  # a few input channels carry most of the activation energy
    col = imatrix.ImatrixCollector()
    lin = col.hook_linear({"model.block.0.mlp.up.weight": w})
    for _ in range(4):
        lin("model.block.0.mlp.up.weight", torch.randn((50, 128), generator=g) * scale)
    col.save(tmp_path / "im.npz")
    im = imatrix.load(tmp_path / "im.npz")
    imp = imatrix.input_importance(im, "model.block.0.mlp.up.weight")
    assert imp.shape == (128,) and imp[:16].mean() > 20 * imp[16:].mean()
    assert im["model.block.0.mlp.up.weight.out"].shape == (64,)
    spec = nint.NintSpec(bits=3, groupsize=32, sub_bits=6)
    plain = nint.dequantize_nint(quantize_nint(w.numpy(), spec))
    weighted = nint.dequantize_nint(quantize_nint(w.numpy(), spec, importance=imp))
    err = lambda a: float((((a - w.numpy()) ** 2) * imp[None]).sum())
    assert err(weighted) < err(plain)


def test_ew_solver_respects_budget_pools_and_importance(tmp_path):
    def tensor(layer, proj):
        experts = []
        for e in range(4):
            experts.append({"expert_id": e, "candidates": [
                {"family": "NINT2", "distortion": 1.0, "effective_bpw": 2.6, "variable_storage_bits": 260},
                {"family": "NINT4", "distortion": 0.2, "effective_bpw": 4.5, "variable_storage_bits": 450},
                {"family": "NVQ3", "distortion": 0.35, "effective_bpw": 3.3, "variable_storage_bits": 300, "pool_key": "d4",
                 "pool_storage_bits": 200}]})
        return {"name": f"model.block.{layer}.mlp.experts.{proj}.weight", "layer": layer, "projection": proj,
                "fixed_storage_bits": 10, "experts": experts}
    cands = {"format": ew_solver.CANDIDATES_FORMAT, "tensors": [tensor(0, "down"), tensor(0, "up")]}
    imp = {"format": ew_solver.IMPORTANCE_FORMAT, "mode": "score",
           "entries": [{"layer": 0, "expert_id": e, "score": s} for e, s in enumerate([10.0, 1.0, 1.0, 0.1])] +
                      [{"layer": 0, "expert_id": 3, "projection": "down", "score": 50.0}]}
    w = ew_solver.importance_weights(imp)
    assert w[(0, 3, "down")] == 50.0 and w[(0, 3, "up")] == 0.1 and w[(0, 0, "gate")] == 10.0
    scheme, report = ew_solver.solve(imp, cands, budget_bits=2 * 10 + 8 * 330)
    assert scheme["format"] == ew_solver.SCHEME_FORMAT and len(scheme["assignments"]) == 8
    assert report["storage_bits"] <= report["budget_bits"]
    fam = {(a["projection"], a["expert_id"]): a["family"] for a in scheme["assignments"]}
    assert fam[("down", 3)] != "NINT2" and fam[("up", 3)] == "NINT2"  # most / least important expert projection
    # exhaustive check of optimality (3^8 assignments, pool cost paid once per tensor that uses it)
    import itertools
    best = None
    for combo in itertools.product(range(3), repeat=8):
        bits, obj = 20.0, 0.0
        for ti, t in enumerate(cands["tensors"]):
            picks = combo[4 * ti : 4 * ti + 4]
            for e, ci in enumerate(picks):
                c = t["experts"][e]["candidates"][ci]
                bits += c["variable_storage_bits"]
                obj += w[(0, e, t["projection"])] * c["distortion"]
            bits += 200 if 2 in picks else 0
        if bits <= 2 * 10 + 8 * 330 and (best is None or obj < best):
            best = obj
    assert abs(report["objective"] - best) < 1e-9
    with pytest.raises(ValueError):
        ew_solver.solve(imp, cands, budget_bits=100)
    ranks = {"format": ew_solver.IMPORTANCE_FORMAT, "mode": "rank", "rank_weighting": "reciprocal",
             "entries": [{"layer": 0, "expert_id": e, "rank": e + 1} for e in range(4)]}
    rw = ew_solver.importance_weights(ranks)
    assert rw[(0, 0, "up")] == 1.0 and rw[(0, 3, "down")] == 0.25
    for name, doc in (("imp.json", imp), ("cand.json", cands), ("budget.json", {"budget_bits": 3000})):
        import json
        (tmp_path / name).write_text(json.dumps(doc))
    rep = ew_solver.solve_files(tmp_path / "imp.json", tmp_path / "cand.json", tmp_path / "budget.json", tmp_path / "scheme.json")
    assert (tmp_path / "scheme.json").exists() and rep["storage_bits"] <= 3000
