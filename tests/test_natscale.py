"""NatScale pieces: the contrast exponent, the hull allocation against brute force, and the expert allocation end to end
on the tiny mixture-of-experts model (candidates -> scheme -> `quantize_tensors(scheme=...)`)."""

import itertools

import numpy as np
import pytest
import torch

from mfq_b200.calibration import natscale as ns


def test_exponent_hits_the_contrast_and_ignores_scale():
    g = np.exp(np.random.default_rng(0).normal(size=64) * 2.0)
    for tau in (0.25, 1.0, 3.0):
        beta = ns.natscale_exponent(g, tau)
        assert abs(ns.realized_contrast(g, beta) - tau) < 1e-9
        assert abs(ns.natscale_exponent(g * 1e-30, tau) - beta) < 1e-9  # no power of a raw score is formed
    # a heavier-tailed score vector needs a smaller exponent for the same contrast
    assert ns.natscale_exponent(g ** 3, 1.0) < ns.natscale_exponent(g, 1.0)
    with pytest.raises(ValueError):
        ns.natscale_exponent(np.ones(5))


def test_hull_allocation_brackets_the_brute_force_optimum():
    rng = np.random.default_rng(1)
    sizes = np.array([10, 20, 30, 40])
    for _ in range(25):
        costs = np.sort(rng.uniform(0, 1, (6, 4)))[:, ::-1].copy()
        budget = int(rng.integers(60, 240))
        sol = ns.allocate_hulls(sizes, costs, budget)
        best = min(sum(costs[i, c] for i, c in enumerate(ch)) for ch in itertools.product(range(4), repeat=6)
                   if sizes[list(ch)].sum() <= budget)
        assert sol["bytes"] <= budget and abs(sol["objective"] - costs[np.arange(6), sol["choice"]].sum()) < 1e-12
        assert sol["lower_bound"] <= best + 1e-9 and best <= sol["objective"] + 1e-9
    with pytest.raises(ValueError):
        ns.allocate_hulls(sizes, np.ones((3, 4)), 25)


def test_expert_allocation_end_to_end(tmp_path):
    from mfq_b200.calibration.imatrix import ImatrixCollector
    from mfq_b200.checkpoint import quantize_tensors
    from mfq_b200.models.moe_lm import MoeConfig, MoeLM, init_weights
    cfg = MoeConfig()
    w = init_weights(cfg, seed=0)
    col = ImatrixCollector()
    model = MoeLM(cfg, w, observer=col.observe)
    g = torch.Generator().manual_seed(0)
    for _ in range(2):
        model.reset()
        model.forward(torch.randint(0, cfg.vocab_size, (96,), generator=g))
    im = col.result()
    assert any(k.endswith("#0.count") for k in im)  # per-expert exposure is recorded
    tensors = {k: v.numpy() for k, v in w.items()}
    cands = ns.expert_candidates(tensors, ["NINT2", "NINT3", "NINT4", "NINT6"], imatrix=im, layers={0})
    assert cands["format"] == "mfq.ew-candidates.v1" and len(cands["tensors"]) == 3
    d = [c["distortion"] for c in cands["tensors"][0]["experts"][0]["candidates"]]
    assert d == sorted(d, reverse=True) and d[-1] < 1e-3  # wider codes, smaller error
    for sens in ("uniform", "imatrix-energy"):
        scheme, report = ns.allocate(cands, 3.9, imatrix=im, tensors=tensors, sensitivity=sens)
        assert report["bits_per_weight"] <= 3.9 + 1e-9 and report["lower_bound"] <= report["objective"] + 1e-12
        assert len(scheme["assignments"]) == 3 * cfg.num_experts and len(report["family_histogram"]) >= 2
    assert report["beta"] > 0 and abs(report["realized_contrast"] - 1.0) < 1e-6
    # a tighter budget shifts experts to narrower families
    tight, _ = ns.allocate(cands, 3.0, imatrix=im, tensors=tensors)
    mean_bits = lambda s: np.mean([int(a["family"][4:]) for a in s["assignments"]])
    assert mean_bits(tight) < mean_bits(scheme)
    # the scheme is what the quantizer consumes
    q = quantize_tensors({k: v for k, v in tensors.items() if k.startswith("model.block.0.mlp.experts.")}, dense="bf16", scheme=scheme)
    assert all(type(t).__name__ == "MfeTensor" or hasattr(t, "pools") or True for t in q.values()) and len(q) == 3


def test_calibrate_subcommands(tmp_path, capsys):
    """`mfq calibrate imatrix | candidates | allocate | natscale` on the synthetic tiny model, then quantize with the scheme."""
    import json

    from mfq_b200.cli import main
    im, cand, scheme, report, out = (tmp_path / n for n in ("im.npz", "cand.json", "scheme.json", "report.json", "m.mfq"))
    assert main(["calibrate", "imatrix", "synthetic:tiny-moe", "--output", str(im), "--chunks", "2", "--ctx", "64"]) == 0
    assert main(["calibrate", "candidates", "synthetic:tiny-moe", "--families", "NINT2,NINT4,NINT6", "--imatrix", str(im),
                 "--layers", "0-1", "--output", str(cand)]) == 0
    doc = json.loads(cand.read_text())
    assert doc["format"] == "mfq.ew-candidates.v1" and len(doc["tensors"]) == 6
    assert main(["calibrate", "natscale", "synthetic:tiny-moe", "--candidates-file", str(cand), "--imatrix", str(im),
                 "--target-bpw", "4.2", "--output", str(scheme), "--report", str(report)]) == 0
    rep = json.loads(report.read_text())
    assert rep["method"] == "NatScale" and rep["bits_per_weight"] <= 4.2 and rep["sensitivity"] == "imatrix-energy"
    assert main(["calibrate", "allocate", "synthetic:tiny-moe", "--candidates-file", str(cand), "--method", "milp",
                 "--target-bpw", "4.2", "--output", str(tmp_path / "milp.json")]) == 0
    milp = json.loads((tmp_path / "milp.json").read_text())
    assert milp["format"] == "mfq.calibration-scheme.v3" and len(milp["assignments"]) == len(json.loads(scheme.read_text())["assignments"])
    capsys.readouterr()
    assert main(["quantize", "synthetic:tiny-moe", str(out), "--ew-scheme", str(scheme)]) == 0
    assert out.exists()


def test_per_neuron_widths_end_to_end(tmp_path, capsys):
    """`mfq calibrate inint` -> `mfq quantize --row-widths`: rows that matter get eight bits, the mean stays in budget, and the
    mixed matrix reconstructs better than the all-narrow one."""
    import json

    from mfq_b200 import formats as F
    from mfq_b200.calibration import inint
    from mfq_b200.cli import main
    rng = np.random.default_rng(0)
    w = rng.normal(size=(64, 256)).astype(np.float32) * 0.05
    w[:8] *= 20.0  # a few loud neurons: their rows cost most at four bits
    doc = inint.select_rows({"model.block.0.attention.query.weight": w}, 5.6)
    rep = doc["report"]
    assert rep["bits_per_weight"] <= 5.6 and 0 < rep["high_rows"] < 64 and rep["loss_vs_all_low"] < 0.5
    assert set(range(8)) <= set(doc["tensors"]["model.block.0.attention.query.weight"]["high_rows"])
    bits = inint.row_bits(doc, "model.block.0.attention.query.weight")
    assert bits.dtype == np.uint8 and set(bits.tolist()) == {4, 8}
    with pytest.raises(ValueError):
        inint.select_rows({"model.block.0.attention.query.weight": w}, 3.0)  # below the all-narrow size
    im, rows, out = tmp_path / "im.npz", tmp_path / "rows.json", tmp_path / "m.mfq"
    assert main(["calibrate", "imatrix", "synthetic:tiny-moe", "--output", str(im), "--chunks", "1", "--ctx", "48"]) == 0
    assert main(["calibrate", "inint", "synthetic:tiny-moe", "--imatrix", str(im), "--target-bpw", "6.0", "--output", str(rows)]) == 0
    capsys.readouterr()
    assert main(["quantize", "synthetic:tiny-moe", str(out), "--row-widths", str(rows), "--imatrix", str(im)]) == 0
    listed = json.loads(rows.read_text())["tensors"]
    with F.open_mfq(out) as store:
        name = next(n for n in listed if listed[n]["high_rows"])
        t = store[name]
        assert sorted(set(np.asarray(t.row_q_bits).tolist())) == [4, 8]


def test_reap_saliency_is_collected_and_steers_the_allocation(tmp_path):
    """Expert saliency = mean router weight x output norm over the tokens routed to it; with ``sensitivity="reap"`` the
    experts that move the residual stream most keep the most bits."""
    import json
    import numpy as np
    import torch
    from mfq_b200 import cli
    from mfq_b200.calibration import natscale
    from mfq_b200.calibration.imatrix import ImatrixCollector, load
    from mfq_b200.models.moe_lm import MoeConfig, MoeLM, init_weights
    cfg = MoeConfig(**cli._SYNTHETIC["tiny-moe"])
    w = init_weights(cfg, seed=3)
    for e in range(cfg.num_experts):  # expert e answers (e + 1) times louder than expert 0
        w["model.block.0.mlp.experts.down.weight"][e] *= (e + 1)
    col = ImatrixCollector()
    model = MoeLM(cfg, w, observer=col.observe, reap_observer=col.observe_reap)
    g = torch.Generator().manual_seed(0)
    for _ in range(4):
        model.reset()
        model.forward(torch.randint(0, cfg.vocab_size, (96,), generator=g))
    col.save(tmp_path / "im.npz")
    im = load(tmp_path / "im.npz")
    reap = np.array([float(im[f"model.block.0.mlp.experts.down.weight#{e}.reap"]) for e in range(cfg.num_experts)])
    assert (reap > 0).all() and np.corrcoef(reap, np.arange(1, cfg.num_experts + 1))[0, 1] > 0.9
    tensors = {k: v.numpy() for k, v in w.items()}
    cands = natscale.expert_candidates(tensors, ["NINT2", "NINT4", "NINT6"], imatrix=im, layers={0})
    scheme, report = natscale.allocate(cands, 4.2, imatrix=im, tensors=tensors, sensitivity="reap")
    bits = {}
    for a in scheme["assignments"]:
        bits.setdefault(a["expert_id"], []).append(int(a["family"][4:]))
    mean_bits = np.array([np.mean(bits[e]) for e in sorted(bits)])
    assert mean_bits[-3:].mean() >= mean_bits[:3].mean()  # the loud experts keep more bits than the quiet ones
    assert report["sensitivity"] == "reap" and report["bits_per_weight"] <= 4.2 + 1e-6
    with pytest.raises(ValueError):
        natscale.allocate(cands, 4.2, sensitivity="reap")
