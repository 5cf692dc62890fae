"""Ternary format: blob round trip, byte compatibility with the reference package (when installed), quantizer quality."""

import numpy as np

from mfq_b200.formats import ternary


def test_round_trip_and_quality():
    rng = np.random.default_rng(0)
    w = rng.standard_normal((48, 100)).astype(np.float32) * np.linspace(0.5, 2.0, 48, dtype=np.float32)[:, None]
    t = ternary.quantize(w, groupsize=24, sub_bits=3)
    blob = ternary.pack(t)
    back = ternary.unpack(blob)
    assert back.shape == (48, 100) and np.array_equal(back.trits, t.trits) and np.array_equal(back.sub, t.sub)
    assert np.array_equal(ternary.dequantize(back), ternary.dequantize(t))
    assert 1.8 < t.bits_per_weight < 2.1
    err = ((ternary.dequantize(t) - w) ** 2).sum() / (w ** 2).sum()
    assert err < 0.22  # the optimum for a Gaussian with one global ternary step is ~0.19
    # columns as neurons
    t1 = ternary.quantize(w, axis=1)
    assert ternary.dequantize(ternary.unpack(ternary.pack(t1))).shape == w.shape


def test_blob_is_byte_compatible_with_the_reference(reference_pkg):
    from mfq.formats import ternary as ref
    from mfq.quantize import ternary_quant
    rng = np.random.default_rng(1)
    w = rng.standard_normal((16, 77)).astype(np.float32)
    mine = ternary.quantize(w, groupsize=24, sub_bits=4)
    blob = ternary.pack(mine)
    theirs = ref.unpack_neuron_ternary(blob)
    assert np.allclose(ternary_quant.dequantize(theirs), ternary.dequantize(mine))
    assert ref.pack_neuron_ternary(theirs) == blob
    # and their blobs load here
    rq = ternary_quant.quantize(w, ref.NEURON_TERNARY_S3)
    got = ternary.unpack(ref.pack_neuron_ternary(rq))
    assert np.allclose(ternary.dequantize(got), ternary_quant.dequantize(rq))
    err_mine = ((ternary.dequantize(ternary.quantize(w)) - w) ** 2).sum()
    err_ref = ((ternary_quant.dequantize(rq) - w) ** 2).sum()
    assert err_mine <= err_ref * 1.1
