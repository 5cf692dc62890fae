"""NPQ0-S / NPQ0-L: round trip, container dtype, rate, and byte equality with the reference package when it is installed."""

import numpy as np
import pytest

from mfq_b200 import formats as F
from mfq_b200.formats import npq0


def _weights(rows=24, cols=104, seed=0):
    return (np.random.default_rng(seed).normal(size=(rows, cols)) * 0.03).astype(np.float32)


@pytest.mark.parametrize("variant", [npq0.NPQ0_S, npq0.NPQ0_L])
def test_round_trip_rate_and_error(variant, tmp_path):
    w = _weights()
    t = npq0.quantize_npq0(w, variant)
    blob = npq0.pack_npq0(t)
    back = npq0.unpack_npq0(blob)
    assert npq0.pack_npq0(back) == blob and np.array_equal(npq0.dequantize_npq0(back), npq0.dequantize_npq0(t))
    code_bits = {"NPQ0-S": 6 / 8 + 2 / 24, "NPQ0-L": 7 / 8 + 3 / 24}[variant.label]
    assert abs(variant.bits_per_weight(4096, 4096, include_tables=False) - code_bits - 16 / 4096) < 1e-3
    err = float(((npq0.dequantize_npq0(t) - w) ** 2).sum() / (w ** 2).sum())
    assert err < {"NPQ0-S": 0.5, "NPQ0-L": 0.36}[variant.label]  # Gaussian rate-distortion bound at these rates: 0.32 / 0.25
    path = tmp_path / "m.mfq"
    F.save(path, F.FileHeader(model_arch="test"), {"model.block.0.mlp.up.weight": t})
    with F.open_mfq(path) as store:
        assert store.dtype("model.block.0.mlp.up.weight") == variant.label
        assert np.array_equal(F.dequantize(store["model.block.0.mlp.up.weight"]), npq0.dequantize_npq0(t))


def test_wider_variant_is_more_accurate_and_bad_blobs_are_refused():
    w = _weights(32, 192, seed=2)
    e = {v.label: float(((npq0.dequantize_npq0(npq0.quantize_npq0(w, v)) - w) ** 2).sum()) for v in (npq0.NPQ0_S, npq0.NPQ0_L)}
    assert e["NPQ0-L"] < e["NPQ0-S"]
    blob = bytearray(npq0.pack_npq0(npq0.quantize_npq0(w, "NPQ0-S")))
    with pytest.raises(ValueError):
        npq0.unpack_npq0(bytes(blob[:-1]))
    blob[4] = 9  # unknown version
    with pytest.raises(ValueError):
        npq0.unpack_npq0(bytes(blob))
    with pytest.raises(ValueError):
        npq0.quantize_npq0(np.zeros((4, 12), np.float32))  # row length not a multiple of 8


def test_bytes_and_values_equal_the_reference_package(reference_pkg):
    from mfq.formats import npq0_l as rl, npq0_s as rs  # type: ignore
    from mfq.quantize.npq0_l import dequantize_npq0_l  # type: ignore
    from mfq.quantize.npq0_s import dequantize_npq0_s  # type: ignore
    w = _weights(16, 104, seed=5)
    for variant, unpack, pack, deq in ((npq0.NPQ0_S, rs.unpack_npq0_s, rs.pack_npq0_s, dequantize_npq0_s),
                                       (npq0.NPQ0_L, rl.unpack_npq0_l, rl.pack_npq0_l, dequantize_npq0_l)):
        t = npq0.quantize_npq0(w, variant)
        blob = npq0.pack_npq0(t)
        theirs = unpack(blob)
        assert pack(theirs) == blob
        assert np.array_equal(deq(theirs), npq0.dequantize_npq0(t))
