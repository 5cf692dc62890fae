"""Run-time layout of packed expert weights: a re-arrangement of the checkpoint's codes that loses nothing."""

import numpy as np
import pytest

from mfq_b200 import formats as F
from mfq_b200.formats import nint
from mfq_b200.ops import packed
from mfq_b200.quantize.nint import quantize_nint


@pytest.mark.parametrize("bits,gs,k", [(2, 24, 96), (3, 24, 200), (4, 24, 520), (5, 32, 256), (6, 24, 130), (7, 32, 64),
                                       (8, 24, 48), (1, 32, 320), (3, 16, 208), (6, 16, 80)])
def test_nint_layout_is_lossless(bits, gs, k):
    rng = np.random.default_rng(bits * 100 + k)
    w = (rng.standard_normal((40, k)) * 0.05).astype(np.float32)
    t = quantize_nint(w, nint.NintSpec(bits=bits, groupsize=gs, sub_bits=6))
    m = packed.pack_nint(t)
    assert m.k_in == k and m.n_out == 40 and m.tiles == 3  # 40 rows of one width: three 16-row tiles, 8 padding rows
    np.testing.assert_array_equal(packed.dequantize(m), nint.dequantize_nint_rows(t))


def test_rows_of_different_widths_are_tiled_by_width():
    rng = np.random.default_rng(3)
    w = (rng.standard_normal((50, 144)) * 0.05).astype(np.float32)
    t = quantize_nint(w, nint.NintSpec(bits=4, groupsize=24, sub_bits=6))
    widths = rng.integers(2, 7, size=50).astype(np.uint8)
    t.q = np.minimum(t.q, ((1 << widths) - 1)[:, None, None]).astype(np.uint8)  # codes must fit the narrower rows
    t.row_q_bits = widths
    m = packed.pack_nint(t, min_units=3)
    assert m.units == 3 and sorted(set(m.tile_bits.tolist())) == sorted(set(widths.tolist()))
    rows = m.out_row.reshape(-1, 16)
    for ti in range(m.tiles):
        live = rows[ti][rows[ti] >= 0]
        assert (widths[live] == m.tile_bits[ti]).all()
    np.testing.assert_array_equal(packed.dequantize(m), nint.dequantize_nint_rows(t))


def test_mxfp4_layout_is_lossless():
    from mfq_b200.formats import mx
    from mfq_b200.quantize.mxfp4 import quantize_mxfp4
    rng = np.random.default_rng(9)
    w = (rng.standard_normal((24, 160)) * 0.05).astype(np.float32)
    t = quantize_mxfp4(w)
    m = packed.pack_mxfp4(t)
    assert m.tiles == 2 and m.units == 2 and (m.tile_bits == packed.MXFP4_BITS).all()
    np.testing.assert_array_equal(packed.dequantize(m), mx.dequantize_mx(t))
