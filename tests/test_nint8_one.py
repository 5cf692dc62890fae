"""NINT8-1 activation blocks (the Q8_1 layout): rounding rule, block sum, torch twin, equality with the reference package."""

import numpy as np
import torch

from mfq_b200.formats.nint8one import fake_quantize_nint8_one, quantize_nint8_one


def test_blocks_by_hand_and_padding():
    x = np.zeros((2, 40), dtype=np.float32)
    x[0, :4] = [127.0, 63.5, -63.5, 0.4]   # step 1: halves round away from zero
    x[1, 32:] = np.linspace(-1, 1, 8)
    b = quantize_nint8_one(x)
    assert b.q.shape == (2, 2, 32) and b.d.shape == (2, 2) and b.reconstructed.shape == (2, 40) and b.reconstructed.dtype == np.float16
    assert b.q[0, 0, :4].tolist() == [127, 64, -64, 0] and float(b.d[0, 0]) == 1.0 and float(b.s[0, 0]) == 127.0
    assert float(b.d[0, 1]) == 0.0 and not b.q[0, 1].any()              # an all-zero block: step 0, codes 0
    assert b.q[1, 1, 0] == -127 and b.q[1, 1, 7] == 127 and not b.q[1, 1, 8:].any()
    err = np.abs(b.reconstructed.astype(np.float32) - x)
    assert err.max() <= 0.5 * 1.0 + 1e-3


def test_torch_twin_and_reference(reference_pkg):
    from mfq.formats.nint8_one import quantize_nint8_one as ref  # type: ignore
    x = (np.random.default_rng(0).normal(size=(3, 5, 70)) * 3).astype(np.float32)
    mine, theirs = quantize_nint8_one(x), ref(x)
    for name in ("q", "d", "s", "reconstructed"):
        assert np.array_equal(getattr(mine, name), getattr(theirs, name)), name
    assert np.array_equal(fake_quantize_nint8_one(torch.from_numpy(x)).numpy(), mine.reconstructed)


def test_eval_kl_under_activation_rounding(tmp_path, capsys):
    from mfq_b200.cli import main
    base = tmp_path / "base.mfq"
    assert main(["quantize", "synthetic:tiny-moe", str(base), "--full-precision"]) == 0
    capsys.readouterr()
    assert main(["eval", "kl", "--model", str(base), "--base", str(base), "--chunks", "1", "--ctx", "32"]) == 0
    same = float(capsys.readouterr().out.split()[0].split("=")[1])
    assert main(["eval", "kl", "--model", str(base), "--base", str(base), "--chunks", "1", "--ctx", "32", "--activation-q8"]) == 0
    rounded = float(capsys.readouterr().out.split()[0].split("=")[1])
    assert same < 1e-9 and 0 < rounded < 1e-2   # int8 activations alone cost a little, far less than any weight format
