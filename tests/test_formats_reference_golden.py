"""Byte compatibility with the reference container, checked against the installed reference package.

Skipped when the reference is not installed; nothing of the reference is imported by the product.
"""

import numpy as np
import pytest

from mfq_b200 import formats as F
from mfq_b200.formats import container, fp8sq, mfe, mx, nint, nvq
from mfq_b200.quantize import quantize_fp8_block, quantize_mxfp4, quantize_nint, quantize_nvq

RNG = np.random.default_rng(3)
W = (RNG.standard_normal((32, 120)) * 0.05).astype(np.float32)


def test_nint_blob_matches_reference(reference_pkg):
    from mfq.formats import io as rio
    from mfq.formats import nint as rnint
    qw = RNG.integers(1, 9, 32).astype(np.uint8)
    kw = RNG.integers(5, 9, 32).astype(np.uint8)
    mine = quantize_nint(W, F.NintSpec(4, 24, 6), row_q_bits=qw, row_sub_bits=kw)
    blob = nint.pack_nint(mine)
    theirs = rio.unpack_nint(blob)
    assert rio.pack_nint(theirs) == blob
    full = rnint.dequantize_tensor(theirs) if hasattr(rnint, "dequantize_tensor") else None
    if full is not None:
        np.testing.assert_allclose(np.asarray(full, dtype=np.float32), F.dequantize(mine), rtol=0, atol=1e-6)


def test_nint_quantizer_tracks_reference(reference_pkg):
    from mfq.formats import nint as rnint
    spec = rnint.NintSpec(bits=4, groupsize=24, sub_bits=6)
    mine = F.dequantize(quantize_nint(W, F.NintSpec(4, 24, 6)))
    ref_rows = np.stack([rnint.dequantize(rnint.quantize(row, spec)) for row in W])
    err_mine = ((mine - W) ** 2).sum()
    err_ref = ((ref_rows - W) ** 2).sum()
    assert err_mine <= err_ref * 1.02


@pytest.mark.parametrize("cb", ["d4_256", "e8_256"])
def test_nvq_blob_matches_reference(reference_pkg, cb):
    from mfq.formats import nvq as rnvq
    from mfq.quantize import nvq_quant
    mine = quantize_nvq(W, F.NvqSpec(cb))
    blob = nvq.pack_nvq(mine)
    theirs = rnvq.unpack_nvq(blob)
    assert rnvq.pack_nvq(theirs) == blob
    np.testing.assert_allclose(nvq_quant.dequantize(theirs), F.dequantize(mine), rtol=0, atol=1e-7)
    ref_q = nvq_quant.quantize(W, rnvq.NvqSpec(cb))
    err_ref = ((nvq_quant.dequantize(ref_q) - W) ** 2).sum()
    err_mine = ((F.dequantize(mine) - W) ** 2).sum()
    assert err_mine <= err_ref * 1.05
    assert np.array_equal(F.dequantize(nvq.unpack_nvq(rnvq.pack_nvq(ref_q))), nvq_quant.dequantize(ref_q))


def test_lattice_grids_match_reference(reference_pkg):
    from mfq.formats import nvq as rnvq
    for name in ("e8_256", "d4_256", "d4_512", "e8_1024", "e8_4096", "d4_1024"):
        assert np.array_equal(nvq.codebook(name), rnvq.codebook_for(rnvq.NvqSpec(name)))


def test_jsc_blob_matches_reference(reference_pkg):
    from mfq.formats import nvq as rnvq
    for cbname, layout in [("d4_256", "streams"), ("e8_4096", "group64"), ("d4_512", "streams")]:
        spec = F.NvqSpec(cbname)
        out, n = 4, 96
        lut, bank = nvq.analytic_jsc_tables(4, spec.vector_size)
        j = F.NvqJscTensor(
            base_spec=spec, shape=(out, n), axis=0, neuron_len=n, neuron_scale=np.ones(out, np.float32), scale_lut=lut,
            bank_for_state=bank, codebooks=np.stack([nvq.codebook(cbname)] * 4),
            state=RNG.integers(0, 16, (out, n // 24)).astype(np.uint8),
            indices=RNG.integers(0, spec.entries, (out, n // spec.vector_size)).astype(np.uint16),
            signs=RNG.integers(0, 128, (out, n // 8)).astype(np.uint8), storage_layout=layout)
        blob = nvq.pack_nvq(j)
        theirs = rnvq.unpack_nvq(blob)
        assert rnvq.pack_nvq(theirs) == blob


def test_mx_fp8_mfe_and_file_match_reference(reference_pkg, tmp_path):
    from mfq.formats import io as rio
    from mfq.formats.header import FileHeader as RefHeader
    w = (RNG.standard_normal((8, 16, 128)) * 0.02).astype(np.float32)
    m4 = quantize_mxfp4(w[0])
    assert rio.pack_mx(rio.unpack_mx("MXFP4", mx.pack_mx(m4))) == mx.pack_mx(m4)
    f8 = quantize_fp8_block(w[1])
    blob8 = fp8sq.pack_fp8sq(f8)
    ref8 = rio.unpack_fp8_sq("FP8-128SQ", blob8)
    assert rio.pack_fp8_sq(ref8) == blob8
    from mfq.formats.fp8_sq import decode_fp8_sq_codes
    assert np.array_equal(decode_fp8_sq_codes(ref8), f8.codes)
    pools = (mfe.MfePool(np.array([0, 3, 5, 6], np.int32), quantize_nint(w[[0, 3, 5, 6]].reshape(64, 128), F.NintSpec())),
             mfe.MfePool(np.array([1, 2, 4, 7], np.int32), quantize_nvq(w[[1, 2, 4, 7]].reshape(64, 128), F.NvqSpec("d4_256"))))
    mt = F.MfeTensor((8, 16, 128), pools)
    tensors = {"model.block.0.mlp.experts.gate.weight": mt, "n": F.to_bf16(np.ones(4, np.float32)), "__mfq_asset__/a": b"xyz"}
    path = tmp_path / "x.mfq"
    container.save(path, F.FileHeader(model_arch="arch", extra={"k": {"v": [1, 2]}}), tensors)
    header, loaded = rio.load(path)
    assert header.model_arch == "arch" and header.extra == {"k": {"v": [1, 2]}}
    assert list(loaded) == list(tensors) and loaded["__mfq_asset__/a"] == b"xyz"
    path2 = tmp_path / "y.mfq"
    rio.save(path2, RefHeader(version=2, model_arch="arch", extra={"k": {"v": [1, 2]}}), loaded)
    assert path.read_bytes() == path2.read_bytes()


def test_nint8_zero_matches_reference(reference_pkg, tmp_path):
    from mfq.formats import nint8_zero as r80
    from mfq_b200.formats import nint8zero
    w = (RNG.standard_normal((24, 96)) * 0.05).astype(np.float32)
    mine = nint8zero.quantize_nint8_zero(w)
    theirs = r80.quantize_nint8_zero(w, axis=0)
    blob = nint8zero.pack_nint8_zero(mine)
    assert blob == r80.pack_nint8_zero(theirs)  # same rule, same bytes
    back = r80.unpack_nint8_zero(blob)
    np.testing.assert_array_equal(np.asarray(back.q), mine.q)
    np.testing.assert_array_equal(F.dequantize(nint8zero.unpack_nint8_zero(blob)), F.dequantize(mine))
    container.save(tmp_path / "z.mfq", container.FileHeader(model_arch="t"), {"model.a.weight": mine})
    with container.open_mfq(tmp_path / "z.mfq") as st:
        assert st.dtype("model.a.weight") == "NINT8-0" and np.array_equal(st["model.a.weight"].q, mine.q)
