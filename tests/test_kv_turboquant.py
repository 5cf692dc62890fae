"""TurboQuant-style KV codec: levels, size, distortion and inner-product preservation."""

import numpy as np
import pytest

from mfq_b200.engine import kv_turboquant as tq


def test_lloyd_max_tables():
    c2, t2 = tq.lloyd_max_gaussian(2)
    assert np.allclose(c2, [-1.510, -0.4528, 0.4528, 1.510], atol=2e-3) and np.allclose(t2, [-0.9816, 0, 0.9816], atol=2e-3)
    c1, _ = tq.lloyd_max_gaussian(1)
    assert np.allclose(np.abs(c1), np.sqrt(2 / np.pi), atol=1e-3)


@pytest.mark.parametrize("bits", [0, 1, 5, 7, 16, "4", float("nan"), float("inf"), True])
def test_invalid_levels_are_rejected(bits):
    with pytest.raises(ValueError):
        tq.validate_bits(bits)


def test_round_trip_size_and_distortion():
    rng = np.random.default_rng(0)
    # keys with a few dominant channels, like real attention keys: the rotation spreads them
    x = rng.standard_normal((512, 128)).astype(np.float32)
    x[:, :4] *= 8.0
    q = rng.standard_normal((64, 128)).astype(np.float32)
    prev = None
    for bits in tq.LEVELS:
        blk = tq.encode(x, bits)
        y = tq.decode(blk)
        assert y.shape == x.shape
        assert blk.nbytes == 512 * 2 + 512 * 128 * bits / 8
        rel = float(((y - x) ** 2).sum() / (x ** 2).sum())
        # theory for the Gaussian Lloyd-Max quantizer: 0.1175 at 2 bits, 0.0345 at 3, 0.0095 at 4, ~4x less per extra bit
        bound = {2: 0.13, 2.5: 0.09, 3: 0.04, 3.5: 0.027, 4: 0.012, 6: 1e-3, 8: 1e-4}[bits]
        assert rel < bound, (bits, rel)
        assert prev is None or rel < prev
        prev = rel
        s_ref, s_got = q @ x.T, q @ y.T
        assert float(np.abs(s_got - s_ref).mean() / np.abs(s_ref).mean()) < 2.5 * np.sqrt(bound)
    # without the rotation the outlier channels would dominate a per-vector quantizer; with it a zero vector is still fine
    z = tq.decode(tq.encode(np.zeros((2, 64), np.float32), 3))
    assert np.all(z == 0)
