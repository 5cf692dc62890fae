"""NVQ-JSC quantizer: trained state scales and codebook banks against the analytic tables and plain NVQ, container round
trip in both storage layouts, expert-mix families, equality with the reference package's reader and decoder."""

import numpy as np
import pytest

from mfq_b200 import formats as F
from mfq_b200.formats.nvq import NvqJscTensor, NvqSpec, analytic_jsc_tables
from mfq_b200.quantize.nvq import quantize_nvq
from mfq_b200.quantize.nvq_jsc import quantize_nvq_jsc


def _w(rows=48, cols=192, seed=0):
    return (np.random.default_rng(seed).standard_t(df=6, size=(rows, cols)) * 0.03).astype(np.float32)


def _rel(t, w):
    return float(((F.dequantize(t) - w) ** 2).sum() / (w ** 2).sum())


@pytest.mark.parametrize("grid,banks", [("e8_256", 1), ("e8_256", 2), ("d4_256", 4)])
def test_training_beats_the_analytic_tables_and_plain_nvq(grid, banks):
    w = _w()
    plain = _rel(quantize_nvq(w, NvqSpec(grid)), w)
    fixed = quantize_nvq_jsc(w, grid, banks=banks, train=False)
    tuned = quantize_nvq_jsc(w, grid, banks=banks)
    lut, bank_map = analytic_jsc_tables(banks, NvqSpec(grid).vector_size)
    assert np.array_equal(fixed.scale_lut, lut) and np.array_equal(fixed.bank_for_state, bank_map) and np.array_equal(tuned.bank_for_state, bank_map)
    assert _rel(fixed, w) < 1.3 * plain                     # same bits, same lattice; identical banks only cost scale steps
    assert _rel(tuned, w) < 0.85 * _rel(fixed, w)           # learned scales + tables pay
    assert tuned.codebooks.shape == (banks, 256, NvqSpec(grid).vector_size) and tuned.codebooks.dtype == np.int8 and tuned.codebooks.min() >= 0
    assert tuned.state.max() <= 15 and np.all(tuned.scale_lut >= 0) and np.array_equal(tuned.scale_lut, tuned.scale_lut.astype(np.float16).astype(np.float32))
    dtype, blob = F.pack_tensor(tuned)
    back = F.unpack_tensor(dtype, blob)
    assert dtype == "NVQ" and isinstance(back, NvqJscTensor) and F.pack_tensor(back)[1] == blob
    assert np.array_equal(F.dequantize(back), F.dequantize(tuned))
    kept = quantize_nvq_jsc(w, grid, banks=banks, learn_scales=False)
    assert np.array_equal(kept.scale_lut, lut) and _rel(kept, w) < _rel(fixed, w)


def test_formula_axis_importance_and_group_records():
    w = _w(16, 72, seed=2)
    t = quantize_nvq_jsc(w.T.copy(), "e8_256", banks=2, axis=1)
    rec = F.dequantize(t)
    assert rec.shape == (72, 16)
    r, g = 3, 2
    s = int(t.state[r, g])
    signs = np.array([-1.0 if (int(t.signs[r, 6 + v]) >> b) & 1 else 1.0 for v in range(3) for b in range(7)]).reshape(3, 7)
    last = np.where(((t.signs[r, 6:9][:, None] >> np.arange(7)) & 1).sum(1) & 1, -1.0, 1.0)
    mags = t.codebooks[t.bank_for_state[s], t.indices[r, 6:9]].astype(np.float32)
    want = t.neuron_scale[r] * t.scale_lut[s] * mags * np.concatenate([signs, last[:, None]], 1)
    assert np.allclose(rec[48:72, r], want.reshape(-1))
    imp = np.ones(192, dtype=np.float32)
    imp[:24] = 50.0
    wide = _w(32, 192, seed=3)
    a, b = quantize_nvq_jsc(wide, "e8_256"), quantize_nvq_jsc(wide, "e8_256", importance=imp)
    err = lambda t: ((F.dequantize(t) - wide)[:, :24] ** 2).sum()
    assert err(b) < err(a)
    xl = quantize_nvq_jsc(_w(8, 96, seed=4), "e8_4096", banks=4, iterations=1, storage_layout="group64")
    dtype, blob = F.pack_tensor(xl)
    back = F.unpack_tensor(dtype, blob)
    assert back.storage_layout == "group64" and np.array_equal(F.dequantize(back), F.dequantize(xl))
    with pytest.raises(ValueError):
        quantize_nvq_jsc(w, "e8_256", banks=3)
    with pytest.raises(ValueError):
        quantize_nvq_jsc(w, NvqSpec("e8_256", groupsize=32))


def test_expert_mix_families():
    from mfq_b200.quantize.expertwise import parse_profiles, quantize_expertwise, quantize_matrix
    t = quantize_matrix(_w(16, 96), parse_profiles("NVQ3J")[0])
    lut, _ = analytic_jsc_tables(2, 4)
    assert isinstance(t, NvqJscTensor) and t.codebooks.shape[0] == 2 and np.array_equal(t.scale_lut, lut)   # NVQ3J keeps the analytic scales
    assert parse_profiles("NVQ2J-XL")[0].nominal_bpw > parse_profiles("NVQ2J")[0].nominal_bpw
    w = np.stack([_w(8, 96, seed=e) for e in range(4)])
    mfe = quantize_expertwise(w, np.array([0, 1, 0, 1]), parse_profiles("NVQ2J,NINT4"))
    rec = F.dequantize(F.unpack_tensor(*F.pack_tensor(mfe)))
    assert rec.shape == w.shape and float(((rec - w) ** 2).sum() / (w ** 2).sum()) < 0.1


def test_reference_package_reads_and_decodes_it(reference_pkg):
    from mfq.formats import nvq as R  # type: ignore
    from mfq.quantize.nvq_jsc import dequantize_nvq_jsc  # type: ignore
    w = _w(12, 96, seed=5)
    for grid, banks, layout in (("e8_256", 2, "streams"), ("d4_256", 1, "streams"), ("e8_4096", 4, "group64")):
        t = quantize_nvq_jsc(w, grid, banks=banks, iterations=1, storage_layout=layout)
        blob = F.pack_tensor(t)[1]
        theirs = R.unpack_nvq(blob)
        assert type(theirs).__name__ == "NvqJscTensor" and R.pack_nvq(theirs) == blob
        assert np.array_equal(dequantize_nvq_jsc(theirs), F.dequantize(t))


def test_tensor_local_codebook_for_plain_nvq(reference_pkg):
    """A codebook fitted to the tensor stays on the format's alphabet, has no repeated entry, travels in the blob, lowers
    the error on rows it was not fitted on, and the reference package reads the result."""
    from mfq.formats import nvq as R  # type: ignore
    from mfq_b200.quantize.nvq import train_tensor_codebook
    rng = np.random.default_rng(7)
    # magnitudes drawn from a small set of shapes the standard grid does not favour
    shapes = rng.choice([1.0, 3.0, 5.0, 7.0], size=(24, 8), p=[0.1, 0.2, 0.3, 0.4])
    rows = []
    for _ in range(160):
        mag = shapes[rng.integers(0, 24, size=24)].reshape(-1)
        rows.append(mag * rng.choice([-1.0, 1.0], size=192) * 0.01 * (1 + 0.03 * rng.normal(size=192)))
    w = np.asarray(rows, dtype=np.float32)
    spec = NvqSpec("e8_256")
    table = train_tensor_codebook(w[:96], spec)
    assert table.shape == (256, 8) and table.dtype == np.int8 and set(np.unique(table).tolist()) <= {1, 3, 5, 7}
    assert np.unique(table, axis=0).shape[0] == 256
    plain, own = quantize_nvq(w[96:], spec), quantize_nvq(w[96:], spec, codebook=table)
    assert _rel_on(own, w[96:]) < 0.7 * _rel_on(plain, w[96:])
    dtype, blob = F.pack_tensor(own)
    back = F.unpack_tensor(dtype, blob)
    assert len(blob) == len(F.pack_tensor(plain)[1]) + 512 and np.array_equal(back.codebook, table)
    assert np.array_equal(F.dequantize(back), F.dequantize(own))
    theirs = R.unpack_nvq(blob)
    assert R.pack_nvq(theirs) == blob


def _rel_on(t, w):
    return float(((F.dequantize(t) - w) ** 2).sum() / (w ** 2).sum())


def test_additive_and_product_vector_code_experiments():
    """15 bits per 8-vector spent as two added codewords or as two half-vector codewords: the rounds only lower the error,
    the tables are int8, and on a heavy-tailed matrix both land below plain NVQ2 (tables fitted to the matrix itself)."""
    from mfq_b200.quantize.nvq_experiments import vector_code_experiment
    w = _w(96, 192, seed=9)
    for kind, shape in (("additive", (256, 8)), ("product", (256, 4))):
        r = vector_code_experiment(w, kind, rounds=4)
        assert r.first.shape == shape and r.second.shape == (128, shape[1]) and r.first.dtype == np.int8
        assert all(b <= a * 1.002 for a, b in zip(r.history, r.history[1:])) and r.rel_error == r.history[-1]
        assert r.rel_error < r.nvq2_rel_error and abs(r.bits_per_weight - (15 / 8 + 4 / 24 + 16 / 192)) < 1e-9
    with pytest.raises(ValueError):
        vector_code_experiment(w[:, :100], "additive")
    with pytest.raises(ValueError):
        vector_code_experiment(w, "lattice")
