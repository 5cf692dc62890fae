"""MXFP4-SQ: palette catalogue, decoding of palette-coded rows, the palette/state search, width allocation, the native
4-bit paths reading it, and agreement with the reference package."""

import json

import numpy as np
import pytest

from mfq_b200 import formats as F
from mfq_b200.formats import mxfp4sq as S
from mfq_b200.formats.mx import dequantize_mx
from mfq_b200.quantize.mxfp4 import quantize_mxfp4
from mfq_b200.quantize.mxfp4_sq import quantize_mxfp4_sq, row_nbytes, select_scale_base

_VAL = np.array([0, 0.5, 1, 1.5, 2, 3, 4, 6, 0, -0.5, -1, -1.5, -2, -3, -4, -6], dtype=np.float64)


def _source(rows=48, cols=256, seed=0):
    w = (np.random.default_rng(seed).standard_t(df=5, size=(rows, cols)) * 0.02).astype(np.float32)
    src = quantize_mxfp4(w)
    return src, dequantize_mx(src)


def _rel(t, full):
    return float(((S.dequantize_mxfp4sq(t) - full) ** 2).sum() / (full ** 2).sum())


def test_catalogue():
    for q in (1, 2, 3):
        p = S.PALETTES[q]
        assert p.shape == (32, 1 << q) and not p.flags.writeable
        vals = _VAL[p]
        assert (np.diff(vals, axis=1) > 0).all()                       # ascending, so distinct values
        assert np.unique(p, axis=0).shape[0] == 32 and not (p == 8).any()  # 32 different palettes, never the negative zero
    assert S.PALETTES[1][:3].tolist() == [[15, 6], [14, 7], [13, 7]]       # (-6, 4), (-4, 6), (-3, 6)
    assert S.PALETTES[2][0].tolist() == [15, 13, 0, 5] and S.PALETTES[3][0].tolist() == [15, 14, 13, 11, 0, 3, 5, 7]
    assert S.PALETTES[2][-2].tolist() == [15, 14, 13, 12]                   # catalogue number 0: the four most negative values


@pytest.mark.parametrize("q", [1, 2, 3])
def test_rows_decode_by_the_state_rule(q):
    src, full = _source(8, 128, seed=q)
    t = quantize_mxfp4_sq(src, row_q_bits=q)
    blob = S.pack_mxfp4sq(t)
    assert len(blob) == 24 + 4 + 8 * 128 * q // 8 + (8 * 4 + 7) // 8 + 8 * 2 + 8 * 5     # header, widths, symbols, 1 + 2*8 + 5*8 bits per row
    back = S.unpack_mxfp4sq(blob)
    assert S.pack_mxfp4sq(back) == blob
    mx = S.to_mxfp4(back)
    r, b = 5, 2
    sym = S.unpack_symbols(back.row_symbols[r], 128, q)[b * 32 : b * 32 + 32]
    if q == 1:
        low = int(np.bitwise_xor.reduce(sym[0::2]) | (np.bitwise_xor.reduce(sym[1::2]) << 1))
    else:
        low = int(np.bitwise_xor.reduce(sym & 3))
    state = low | (int(back.block_selectors[r, b]) << 2)
    assert int(mx.scales[r, b]) == back.matrix_scale_base + int(back.state_scales[r, state])
    nib = S.PALETTES[q][int(back.state_palettes[r, state])][sym]
    got = np.asarray(mx.values[r, b * 16 : b * 16 + 16])
    assert np.array_equal(got & 15, nib[0::2]) and np.array_equal(got >> 4, nib[1::2])
    want = _VAL[nib] * 2.0 ** (int(mx.scales[r, b]) - 127)
    assert np.allclose(S.dequantize_mxfp4sq(back)[r, b * 32 : b * 32 + 32], want)
    # every compressed block sits in the four-exponent window
    assert mx.scales.min() >= back.matrix_scale_base and mx.scales.max() <= back.matrix_scale_base + 3


def test_error_falls_with_width_and_q4_is_the_source():
    src, full = _source()
    errs = {q: _rel(quantize_mxfp4_sq(src, row_q_bits=q), full) for q in (1, 2, 3, 4)}
    assert errs[4] == 0.0 and errs[3] < 0.05 and errs[2] < 0.16 and errs[1] < 0.5 and errs[1] > errs[2] > errs[3]
    t = quantize_mxfp4_sq(src, row_q_bits=4)
    mx = S.to_mxfp4(t)
    assert np.array_equal(mx.values, src.values) and np.array_equal(mx.scales, src.scales) and t.is_native
    # eight states beat one: the same rows forced through a single palette and exponent are clearly worse
    from mfq_b200.quantize import mxfp4_sq as Q
    one = Q._choose_states
    try:
        Q._choose_states = lambda err: np.repeat(err.sum(1).argmin(1)[:, None], 8, axis=1)
        single = _rel(quantize_mxfp4_sq(src, row_q_bits=2), full)
    finally:
        Q._choose_states = one
    assert errs[2] < 0.8 * single


def test_mixed_widths_and_allocation():
    src, full = _source(32, 256, seed=3)
    q = np.array([1, 2, 3, 4] * 8)
    t = quantize_mxfp4_sq(src, row_q_bits=q)
    blob = S.pack_mxfp4sq(t)
    back = S.unpack_mxfp4sq(blob)
    assert np.array_equal(back.row_q_bits, q) and back.block_selectors.shape == (24, 8) and back.native_scales.shape == (8, 8)
    rec = S.dequantize_mxfp4sq(back)
    assert np.array_equal(rec[3::4], full[3::4])
    per_row = ((rec - full) ** 2).sum(1)
    assert per_row[0::4].mean() > per_row[1::4].mean() > per_row[2::4].mean() > 0
    # a mean-bits target is met (to the granularity of one row) and the error falls as the budget grows
    last = None
    for bits in (1.6, 2.5, 3.4, 4.25):
        a = quantize_mxfp4_sq(src, target_bits=bits)
        stored = 8.0 * sum(row_nbytes(int(x), 256) for x in a.row_q_bits) / full.size
        assert stored <= bits + 1e-9 and stored > bits - 8.0 * (row_nbytes(4, 256) - row_nbytes(3, 256)) / 256 / 32 - 0.3
        e = _rel(a, full)
        assert last is None or e <= last
        last = e
    assert last == 0.0
    # important rows keep more bits
    imp = np.ones(32)
    imp[:8] = 100.0
    a = quantize_mxfp4_sq(src, target_bits=2.5, importance=imp)
    assert a.row_q_bits[:8].mean() > a.row_q_bits[8:].mean()
    with pytest.raises(ValueError):
        quantize_mxfp4_sq(src)
    with pytest.raises(ValueError):
        quantize_mxfp4_sq(src, row_q_bits=5)


def test_exponent_window_choice():
    src, _ = _source(16, 128, seed=4)
    nib = np.empty((16, 128), dtype=np.uint8)
    nib[:, 0::2], nib[:, 1::2] = src.values & 15, src.values >> 4
    base = select_scale_base(nib, src.scales)
    s = src.scales.astype(int)
    inside = ((s >= base) & (s <= base + 3)).mean()
    assert inside > 0.9 and base <= int(np.median(s)) <= base + 3


def test_native_4bit_paths_read_palette_rows():
    from mfq_b200.ops import w4 as w4ops
    from mfq_b200.ops.packed import _expert_slice
    src, _ = _source(32, 256, seed=5)
    t = quantize_mxfp4_sq(src, target_bits=2.5)
    mx = S.to_mxfp4(t)
    a, b = w4ops.from_checkpoint_tensor(t), w4ops.from_checkpoint_tensor(mx)
    assert a is not None and np.array_equal(w4ops.dequantize(a).numpy(), w4ops.dequantize(b).numpy())
    assert np.allclose(w4ops.dequantize(a).numpy(), S.dequantize_mxfp4sq(t), rtol=1e-2, atol=1e-6)   # bf16-rounded scales are exact powers of two
    part = _expert_slice(t, 1, 16)
    assert np.array_equal(part.values, mx.values[16:32]) and np.array_equal(part.scales, mx.scales[16:32])
    assert S.expanded(t) is S.expanded(t)


def test_cli_recodes_dense_and_expert_matrices(tmp_path, capsys):
    import torch
    from mfq_b200.checkpoint import load_engine
    from mfq_b200.cli import main
    base, plain, sq = tmp_path / "base.mfq", tmp_path / "mx.mfq", tmp_path / "sq.mfq"
    assert main(["quantize", "synthetic:tiny-moe-128", str(base), "--full-precision"]) == 0
    assert main(["quantize", "synthetic:tiny-moe-128", str(plain), "--format", "mxfp4"]) == 0
    assert main(["quantize", "synthetic:tiny-moe-128", str(sq), "--format", "mxfp4", "--mxfp4-sq-bits", "3.0"]) == 0
    capsys.readouterr()
    assert main(["inspect", str(sq)]) == 0
    info = json.loads(capsys.readouterr().out)
    assert "MXFP4-SQ" in info["bytes_by_dtype"] and "MXFP4" not in info["bytes_by_dtype"]
    assert sq.stat().st_size < 0.85 * plain.stat().st_size
    with F.open_mfq(sq) as store:
        name = next(n for n in store if n.endswith("mlp.experts.down.weight"))
        assert all(isinstance(p.tensor, S.Mxfp4SqTensor) for p in store[name].pools)
    assert main(["eval", "kl", "--model", str(sq), "--base", str(base), "--chunks", "2", "--ctx", "64"]) == 0
    line = capsys.readouterr().out.strip()
    assert float(line.split()[0].split("=")[1]) < 0.05, line
    engine, tok, _cfg = load_engine(sq, "cpu", max_batch=2, max_seq_len=64)
    assert engine.generate([torch.tensor(tok.encode("hello"))], 4).tokens.shape == (1, 4)


def test_agrees_with_the_reference_package(reference_pkg):
    from mfq.formats.mxfp4_sq import unpack_mxfp4_sq  # type: ignore
    from mfq.quantize.mxfp4_sq import SQ1_PALETTE_NIBBLES, SQ2_PALETTE_NIBBLES, SQ3_PALETTE_NIBBLES, quantize_mxfp4_sq as ref_q  # type: ignore
    assert np.array_equal(SQ1_PALETTE_NIBBLES, S.PALETTES[1]) and np.array_equal(SQ2_PALETTE_NIBBLES, S.PALETTES[2])
    assert np.array_equal(SQ3_PALETTE_NIBBLES, S.PALETTES[3])
    src, full = _source(24, 256, seed=6)
    for q in (2, 3, np.array([1] + [2, 3, 4] * 7 + [2, 3])):  # one row of width 1: their solver for it is slow without numba
        mine = quantize_mxfp4_sq(src, row_q_bits=q)
        theirs = ref_q(np.asarray(src.values), np.asarray(src.scales), row_q_bits=q, matrix_scale_base=mine.matrix_scale_base)
        blob = S.pack_mxfp4sq(mine)
        assert len(blob) == len(theirs.payload)
        assert unpack_mxfp4_sq(blob).row_q_bits == tuple(int(x) for x in mine.row_q_bits)   # their reader accepts our payload
        read = S.unpack_mxfp4sq(theirs.payload)                                               # and ours theirs, byte for byte
        assert S.pack_mxfp4sq(read) == theirs.payload
        assert _rel(mine, full) <= 1.03 * _rel(read, full)
    ref_auto = ref_q(np.asarray(src.values), np.asarray(src.scales), row_q_bits=2)
    assert quantize_mxfp4_sq(src, row_q_bits=2).matrix_scale_base == ref_auto.matrix_scale_base
