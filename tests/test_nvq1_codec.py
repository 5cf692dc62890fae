"""NVQ1-L / NVQ1-S: layout, round trip, encoder quality, container dtype, byte equality with the reference package."""

import math
import struct

import numpy as np
import pytest

from mfq_b200 import formats as F
from mfq_b200.formats import nvq1


def _weights(rows=12, cols=96, seed=0):
    return (np.random.default_rng(seed).normal(size=(rows, cols)) * 0.04).astype(np.float32)


def test_grid_is_the_ternary_iq1s_table():
    g = nvq1.IQ1S_GRID
    assert g.shape == (2048, 8) and set(np.unique(g).tolist()) == {-1, 0, 1}
    assert np.unique(g, axis=0).shape[0] == 2048 and not g.flags.writeable
    assert nvq1._pack_table(g, 2048) == (nvq1.Path(nvq1.__file__).parent / "data" / "iq1s_grid.bin").read_bytes()


@pytest.mark.parametrize("name", ["NVQ1-L", "NVQ1-L-S4", "NVQ1-S"])
def test_round_trip_layout_and_error(name, tmp_path):
    w = _weights()
    t = nvq1.quantize_nvq1(w, name)
    v = t.variant
    blob = nvq1.pack_nvq1(t)
    # header and stream sizes as the format defines them
    magic, second, sub_bits, gs, axis, row_len, ndim = struct.unpack_from("<4sBBHiiI", blob)
    assert magic == v.magic and sub_bits == v.sub_bits and gs == 24 and (axis, row_len, ndim) == (0, 96, 2) and second == 1
    table = 2048 if v.banked else 0
    assert len(blob) == 20 + 16 + 4 + table + v.stream_nbytes(12, 96)
    code_bits = (3 * v.index_bits + v.sub_bits + 1) / 24
    assert abs(v.bits_per_weight(4096, 4096, include_table=False) - code_bits - 16 / 4096) < 1e-3
    back = nvq1.unpack_nvq1(blob)
    assert nvq1.pack_nvq1(back) == blob and np.array_equal(nvq1.dequantize_nvq1(back), nvq1.dequantize_nvq1(t))
    rec = nvq1.dequantize_nvq1(t)
    err = float(((rec - w) ** 2).sum() / (w ** 2).sum())
    assert err < {"NVQ1-L": 0.22, "NVQ1-L-S4": 0.22, "NVQ1-S": 0.30}[name], err  # Gaussian bound at 1.5 / 1.33 bits: 0.12 / 0.16
    path = tmp_path / "m.mfq"
    F.save(path, F.FileHeader(model_arch="test"), {"model.block.0.mlp.up.weight": t})
    with F.open_mfq(path) as store:
        assert store.dtype("model.block.0.mlp.up.weight") == v.label
        assert np.array_equal(F.dequantize(store["model.block.0.mlp.up.weight"]), rec)


def test_formula_short_groups_axis_and_importance():
    # the reconstruction formula, by hand, including a short last group (row length 40 = 24 + 16) and axis 1
    w = _weights(7, 40, seed=3)
    t = nvq1.quantize_nvq1(w.T.copy(), "NVQ1-L", axis=1)
    assert t.shape == (40, 7) and t.sub_scale.shape == (7, 2) and t.indices.shape == (7, 5)
    rec = nvq1.dequantize_nvq1(t)
    assert rec.shape == (40, 7)
    r, vec = 3, 4  # vector 4 lies in group 1
    want = t.anchors[r] * t.sub_scale[r, 1] * (nvq1.IQ1S_GRID[t.indices[r, vec]] + (-0.125 if t.sign[r, 1] else 0.125))
    assert np.allclose(rec[32:40, r], want)
    # importance moves the error to the unimportant columns
    w = _weights(16, 96, seed=4)
    imp = np.ones(96, dtype=np.float32)
    imp[:24] = 100.0
    plain, weighted = nvq1.quantize_nvq1(w, "NVQ1-L"), nvq1.quantize_nvq1(w, "NVQ1-L", importance=imp)
    e = lambda t: float(((nvq1.dequantize_nvq1(t) - w)[:, :24] ** 2).sum())
    assert e(weighted) <= e(plain) * 1.001
    # more search (iterations) never hurts; NVQ1-S trains its own banks and they stay valid
    s0 = nvq1.quantize_nvq1(w, "NVQ1-S", iterations=1, table_steps=0)
    s2 = nvq1.quantize_nvq1(w, "NVQ1-S", iterations=3, table_steps=2)
    err = lambda t: float(((nvq1.dequantize_nvq1(t) - w) ** 2).sum())
    assert err(s2) <= err(s0) * 1.02
    assert s2.table.shape == (2, 512, 8) and np.unique(s2.table[0], axis=0).shape[0] == 512


def test_own_table_profile_and_refusals():
    w = _weights(4, 48, seed=6)
    t = nvq1.quantize_nvq1(w, "NVQ1-L")
    t.table = nvq1.IQ1S_GRID[::-1].copy()  # a tensor-local table: profile 2, 4096 more bytes, indices mean other entries
    blob = nvq1.pack_nvq1(t)
    assert blob[4] == 2 and len(blob) == len(nvq1.pack_nvq1(nvq1.quantize_nvq1(w, "NVQ1-L"))) + 4096
    back = nvq1.unpack_nvq1(blob)
    assert np.array_equal(back.table, t.table) and np.array_equal(nvq1.dequantize_nvq1(back), nvq1.dequantize_nvq1(t))
    with pytest.raises(ValueError):
        nvq1.unpack_nvq1(blob[:-1])
    with pytest.raises(ValueError):
        nvq1.unpack_nvq1(b"XXXX" + blob[4:])
    with pytest.raises(ValueError):
        nvq1.quantize_nvq1(_weights(4, 20), "NVQ1-S")  # rows of NVQ1-S are a multiple of 8 long
    bad = nvq1.quantize_nvq1(w, "NVQ1-L")
    bad.indices[0, 0] = 2048
    with pytest.raises(ValueError):
        nvq1.pack_nvq1(bad)


def test_expert_mix_accepts_the_family():
    from mfq_b200.quantize.expertwise import parse_profiles, quantize_matrix
    t = quantize_matrix(_weights(8, 48), parse_profiles("NVQ1-S")[0])
    assert isinstance(t, nvq1.Nvq1Tensor) and F.pack_tensor(t)[0] == "NVQ1-S"


def test_bytes_and_values_equal_the_reference_package(reference_pkg):
    from mfq.formats import nvq1_l as rl, nvq1_s as rs  # type: ignore
    from mfq.quantize.nvq1_l_quant import dequantize as deq_l  # type: ignore
    w = _weights(8, 72, seed=9)
    t = nvq1.quantize_nvq1(w, "NVQ1-L")
    blob = nvq1.pack_nvq1(t)
    theirs = rl.unpack_nvq1_l(blob)
    assert rl.pack_nvq1_l(theirs) == blob and np.array_equal(deq_l(theirs), nvq1.dequantize_nvq1(t))
    assert np.array_equal(rl.IQ1S_TERNARY_2048, nvq1.IQ1S_GRID)
    s = nvq1.quantize_nvq1(w, "NVQ1-S")
    sblob = nvq1.pack_nvq1(s)
    theirs = rs.unpack_nvq1_s(sblob)
    assert rs.pack_nvq1_s(theirs) == sblob


def test_tensor_local_table_is_kept_only_when_it_helps():
    rng = np.random.default_rng(11)
    # weights whose 8-vectors come from a small set of patterns the IQ1_S grid does not contain: a trained table wins
    patterns = rng.choice([-1.0, 0.0, 1.0], size=(40, 8), p=[0.45, 0.1, 0.45])
    rows = []
    for _ in range(64):
        pick = patterns[rng.integers(0, 40, size=12)].reshape(-1)
        rows.append(pick * 0.05 * (1 + 0.05 * rng.normal(size=96)))
    w = np.asarray(rows, dtype=np.float32)
    plain = nvq1.quantize_nvq1(w, "NVQ1-L")
    tuned = nvq1.quantize_nvq1(w, "NVQ1-L", train_table=True)
    err = lambda t: float(((nvq1.dequantize_nvq1(t) - w) ** 2).sum())
    assert tuned.table is not None and tuned.table.shape == (2048, 8) and err(tuned) < 0.8 * err(plain), (err(tuned), err(plain))
    assert np.unique(tuned.table, axis=0).shape[0] == 2048 and set(np.unique(tuned.table).tolist()) <= {-1, 0, 1}
    blob = nvq1.pack_nvq1(tuned)
    assert blob[4] == 2 and np.array_equal(nvq1.dequantize_nvq1(nvq1.unpack_nvq1(blob)), nvq1.dequantize_nvq1(tuned))
    # Gaussian weights: the grid is already a good table, the trained one is dropped unless it wins on held-out rows
    g = _weights(48, 96, seed=12)
    t = nvq1.quantize_nvq1(g, "NVQ1-L", train_table=True)
    assert t.table is None or err_of(t, g) <= err_of(nvq1.quantize_nvq1(g, "NVQ1-L"), g) * 1.05


def err_of(t, w):
    return float(((nvq1.dequantize_nvq1(t) - w) ** 2).sum())
