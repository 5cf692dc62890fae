"""Quantizer behaviour beyond round trips: importance-weighted searches."""
def test_importance_weighted_nint_lowers_the_weighted_error():
    """With an imatrix the NINT search minimizes the importance-weighted error of what is stored: it must not be worse
    than the weight-only encoding on that objective, and the stored-format refinement never raises it."""
    import numpy as np
    import torch
    from mfq_b200.formats import nint
    from mfq_b200.quantize.nint import importance_weights, quantize_nint
    rng = np.random.default_rng(11)
    w = (rng.standard_normal((48, 600)) * 0.05).astype(np.float32)
    imp = (rng.random(600) ** 4 * 10 + 0.01).astype(np.float32)  # a few inputs matter far more than the rest
    spec = nint.NintSpec(bits=3, groupsize=24, sub_bits=6)
    plain = nint.dequantize_nint_rows(quantize_nint(w, spec))
    weighted = nint.dequantize_nint_rows(quantize_nint(w, spec, importance=imp))
    ew = importance_weights(torch.from_numpy(w), torch.from_numpy(imp)[None]).numpy()
    err_plain = float((ew * (plain - w) ** 2).sum())
    err_weighted = float((ew * (weighted - w) ** 2).sum())
    assert err_weighted < err_plain, (err_weighted, err_plain)


def test_fp8_sq_palettes_are_exact_and_rows_meet_the_budget():
    import numpy as np
    from mfq_b200 import formats as F
    from mfq_b200.formats.fp8sq import palette_slice, pack_fp8sq, unpack_fp8sq, dequantize_fp8sq
    from mfq_b200.quantize.fp8_block import quantize_fp8_block
    from mfq_b200.quantize.fp8_sq import fit_palette, quantize_fp8_sq
    rng = np.random.default_rng(2)
    w = (rng.standard_normal((256, 256)) * 0.05).astype(np.float32)
    t = quantize_fp8_block(w)
    # a one-bit palette of a two-valued matrix is exact; a fitted palette never loses to a uniform pick of levels
    two = np.where(rng.random((8, 64)) < 0.5, np.uint8(0x38), np.uint8(0xB8))
    assert set(fit_palette(two, None, 1).tolist()) == {0x38, 0xB8}
    pal3 = fit_palette(t.codes, None, 3)
    assert np.unique(pal3).size == 8
    sq = quantize_fp8_sq(t, target_bits=5.0)
    widths = sq.q_widths().astype(np.float64)
    assert abs(widths.mean() - 5.0) < 0.02 and widths.min() >= 1 and widths.max() <= 8
    for q in range(1, 8):  # every row's codes come from its palette
        rows = sq.codes[sq.q_widths() == q]
        assert np.isin(rows, sq.palettes[palette_slice(q)]).all()
    back = unpack_fp8sq("FP8-128SQ", pack_fp8sq(sq))
    np.testing.assert_array_equal(back.codes, sq.codes)
    full, low = dequantize_fp8sq(t), dequantize_fp8sq(sq)
    rel = np.sqrt(((full - low) ** 2).mean()) / np.sqrt((full ** 2).mean())
    assert rel < 0.12, rel  # five bits of a 3-bit-mantissa format: a few percent
    assert len(pack_fp8sq(sq)) < 0.7 * len(pack_fp8sq(t))
