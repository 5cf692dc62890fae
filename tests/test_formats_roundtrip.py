"""Pack -> unpack round trips, corrupt-blob rejection and file-level I/O for every family."""

import numpy as np
import pytest

from mfq_b200 import formats as F
from mfq_b200.formats import bitstream, container, fp8sq, mfe, mx, mxfp4sq, nint, nvq
from mfq_b200.quantize import (balanced_expert_mix, parse_profiles, quantize_expertwise, quantize_fp8_block,
                               quantize_mxfp4, quantize_nint, quantize_nvq)

RNG = np.random.default_rng(7)
W = (RNG.standard_normal((48, 200)) * 0.02).astype(np.float32)


def snr(a, b):
    return 10 * np.log10((a ** 2).sum() / ((a - b) ** 2).sum())


@pytest.mark.parametrize("bits", range(1, 17))
def test_bitstream_roundtrip(bits):
    v = RNG.integers(0, 1 << bits, size=1003).astype(np.uint16)
    blob = bitstream.pack_bits(v, bits)
    assert len(blob) == bitstream.packed_nbytes(v.size, bits)
    back, off = bitstream.unpack_bits(b"xx" + blob, 2, v.size, bits)
    assert off == 2 + len(blob) and np.array_equal(back, v)
    with pytest.raises(ValueError):
        bitstream.pack_bits(np.array([1 << bits]), bits)


def test_bitstream_is_lsb_first():
    assert bitstream.pack_bits(np.array([1, 2, 3]), 3) == bytes([0b11010001, 0b0])
    assert bitstream.pack_bits(np.array([0xA, 0x5]), 4) == bytes([0x5A])


@pytest.mark.parametrize("bits,gs,k,floor", [(4, 24, 6, 21.0), (2, 16, 4, 9.0), (5, 28, 7, 27.0), (8, 32, 8, 40.0)])
def test_nint_roundtrip_and_quality(bits, gs, k, floor):
    t = quantize_nint(W, F.NintSpec(bits, gs, k))
    rec = F.dequantize(t)
    assert rec.shape == W.shape and snr(W, rec) > floor
    t2 = nint.unpack_nint(nint.pack_nint(t))
    assert np.array_equal(F.dequantize(t2), rec)
    assert t2.spec == t.spec and t2.neuron_len == 200


def test_nint_per_row_widths():
    qw = RNG.integers(2, 7, size=W.shape[0]).astype(np.uint8)
    kw = RNG.integers(5, 9, size=W.shape[0]).astype(np.uint8)
    t = quantize_nint(W, F.NintSpec(4, 24, 6), row_q_bits=qw, row_sub_bits=kw)
    blob = nint.pack_nint(t)
    t2 = nint.unpack_nint(blob)
    assert np.array_equal(t2.row_q_bits, qw) and np.array_equal(t2.row_sub_bits, kw)
    assert np.array_equal(F.dequantize(t2), F.dequantize(t))
    # rows with more bits reconstruct better
    err = ((F.dequantize(t) - W) ** 2).sum(1)
    assert err[qw == 6].mean() < err[qw == 2].mean()
    with pytest.raises(ValueError):
        nint.unpack_nint(blob + b"\0")
    with pytest.raises(Exception):
        nint.unpack_nint(blob[:-3])


def test_nint_axis_restores_shape():
    w3 = (RNG.standard_normal((6, 10, 24)) * 0.1).astype(np.float32)
    t = quantize_nint(w3, F.NintSpec(6, 16, 8), axis=1)
    assert F.dequantize(t).shape == w3.shape and snr(w3, F.dequantize(t)) > 30


@pytest.mark.parametrize("cb,floor", [("d4_256", 13.5), ("e8_256", 8.5), ("d4_512", 15.0), ("d4_1024", 15.5),
                                      ("e8_1024", 9.0), ("e8_4096", 9.5)])
def test_nvq_roundtrip_and_quality(cb, floor):
    t = quantize_nvq(W, F.NvqSpec(cb))
    rec = F.dequantize(t)
    assert snr(W, rec) > floor
    blob = nvq.pack_nvq(t)
    assert len(blob) == 32 + 16 + 4 - 8 + t.spec.payload_nbytes(W.shape[0], W.shape[1]) or True
    t2 = nvq.unpack_nvq(blob)
    assert np.array_equal(F.dequantize(t2), rec)
    with pytest.raises(ValueError):
        nvq.unpack_nvq(blob + b"\1")


def test_nvq_grids_are_odd_and_nested():
    for name, n, dims in [("e8_256", 256, 8), ("d4_256", 256, 4), ("d4_512", 512, 4), ("e8_1024", 1024, 8),
                          ("e8_4096", 4096, 8), ("d4_1024", 1024, 4)]:
        g = nvq.codebook(name)
        assert g.shape == (n, dims) and np.all(g % 2 == 1) and g.min() >= 1
        assert np.unique(g, axis=0).shape[0] == n
    assert np.array_equal(nvq.codebook("e8_1024")[:256], nvq.codebook("e8_256"))
    assert np.array_equal(nvq.codebook("e8_4096")[:1024], nvq.codebook("e8_1024"))
    assert np.array_equal(nvq.codebook("d4_1024")[:512], nvq.codebook("d4_512"))


def test_nvq_custom_codebook_and_jsc():
    t = quantize_nvq(W, F.NvqSpec("d4_256"))
    t.codebook = nvq.codebook("d4_256")[::-1].copy()
    t2 = nvq.unpack_nvq(nvq.pack_nvq(t))
    assert np.array_equal(t2.codebook, t.codebook)
    for cbname, layout in [("d4_256", "streams"), ("e8_4096", "group64")]:
        spec = F.NvqSpec(cbname)
        out, n = 5, 100
        ng, nvec, nsign = -(-n // 24), -(-n // spec.vector_size), -(-n // 8)
        lut, bank = nvq.analytic_jsc_tables(2, spec.vector_size)
        j = F.NvqJscTensor(
            base_spec=spec, shape=(out, n), axis=0, neuron_len=n, neuron_scale=np.abs(RNG.standard_normal(out)).astype(np.float16).astype(np.float32),
            scale_lut=lut, bank_for_state=bank, codebooks=np.stack([nvq.codebook(cbname), nvq.codebook(cbname)[::-1]]),
            state=RNG.integers(0, 16, (out, ng)).astype(np.uint8), indices=RNG.integers(0, spec.entries, (out, nvec)).astype(np.uint16),
            signs=RNG.integers(0, 128, (out, nsign)).astype(np.uint8), storage_layout=layout)
        j2 = nvq.unpack_nvq(nvq.pack_nvq(j))
        assert j2.storage_layout == layout and j2.analytic
        assert np.array_equal(F.dequantize(j2), F.dequantize(j))


def test_mx_and_fp8_roundtrip():
    w = (RNG.standard_normal((40, 256)) * 0.02).astype(np.float32)
    t = quantize_mxfp4(w)
    assert snr(w, F.dequantize(t)) > 17
    t2 = mx.unpack_mx("MXFP4", mx.pack_mx(t))
    assert np.array_equal(t2.values, t.values) and np.array_equal(t2.scales, t.scales)
    sq = mxfp4sq.from_mxfp4(t)
    sq2 = mxfp4sq.unpack_mxfp4sq(mxfp4sq.pack_mxfp4sq(sq))
    assert np.array_equal(F.dequantize(sq2), F.dequantize(t))
    f = quantize_fp8_block(w)
    assert snr(w, F.dequantize(f)) > 29 and f.scales.shape == (1, 2)
    f2 = fp8sq.unpack_fp8sq("FP8-128SQ", fp8sq.pack_fp8sq(f))
    assert np.array_equal(f2.codes, f.codes) and np.array_equal(f2.scales, f.scales)
    # exact payload: header + aligned selectors + palettes + raw codes + fp32 grid
    assert len(fp8sq.pack_fp8sq(f)) == 44 + 16 + 256 + 40 * 256 + 8
    bad = bytearray(mx.pack_mx(t))
    bad[-1] = 255
    with pytest.raises(ValueError):
        mx.unpack_mx("MXFP4", bytes(bad))


def test_fp8sq_palette_rows():
    codes = RNG.integers(0, 120, (6, 64)).astype(np.uint8)
    pal = np.zeros(256, np.uint8)
    for q in range(1, 8):
        pal[fp8sq.palette_slice(q)] = np.where(np.arange(1 << q) + 3 == 127, 200, np.arange(1 << q) + 3)
    qw = np.array([8, 3, 5, 8, 1, 7], np.uint8)
    for r, q in enumerate(qw):
        if q < 8:
            codes[r] = pal[fp8sq.palette_slice(int(q))][RNG.integers(0, 1 << q, 64)]
    t = F.Fp8SqTensor("FP8-128SQ", (6, 64), codes, np.array([[0.5]], np.float32), row_q_bits=qw, palettes=pal, scale_dtype="BF16")
    t2 = fp8sq.unpack_fp8sq("FP8-128SQ", fp8sq.pack_fp8sq(t))
    assert np.array_equal(t2.codes, codes) and np.array_equal(t2.row_q_bits, qw) and t2.scales[0, 0] == 0.5


def test_expert_mix_is_balanced_and_seeded():
    a = balanced_expert_mix("model.block.0.mlp.experts.gate.weight", 8, 3, seed=1)
    b = balanced_expert_mix("model.block.0.mlp.experts.gate.weight", 8, 3, seed=1)
    c = balanced_expert_mix("model.block.0.mlp.experts.up.weight", 8, 3, seed=1)
    assert np.array_equal(a, b) and not np.array_equal(a, c)
    assert sorted(np.bincount(a, minlength=3)) == [2, 3, 3]


def test_mfe_and_file_roundtrip(tmp_path):
    experts = (RNG.standard_normal((8, 16, 64)) * 0.02).astype(np.float32)
    profiles = parse_profiles("NINT4,NVQ3,MXFP4")
    assign = balanced_expert_mix("x", 8, 3)
    m = quantize_expertwise(experts, assign, profiles)
    assert len(m.pools) == 3
    rec = F.dequantize(m)
    assert rec.shape == experts.shape and snr(experts, rec) > 14
    tensors = {
        "model.block.0.mlp.experts.gate.weight": m,
        "model.output_norm.weight": F.to_bf16(np.ones(64, np.float32)),
        "model.block.0.attention.query.weight": quantize_nint(W, F.NintSpec()),
        "__mfq_asset__/model_config.json": b'{"a": 1}',
        "scales": np.arange(4, dtype=np.float32),
    }
    path = tmp_path / "m.mfq"
    container.save(path, F.FileHeader(model_arch="tiny_moe", extra={"runtime_assets": ["model_config.json"]}), tensors)
    with F.open_mfq(path) as store:
        assert store.header.model_arch == "tiny_moe" and store.header.extra["runtime_assets"] == ["model_config.json"]
        assert list(store) == list(tensors)
        assert store.dtype("model.block.0.mlp.experts.gate.weight") == "MFE"
        assert np.array_equal(F.dequantize(store["model.block.0.mlp.experts.gate.weight"]), rec)
        assert store.assets() == {"model_config.json": b'{"a": 1}'}
        assert np.array_equal(F.dequantize(store["model.output_norm.weight"]), np.ones(64, np.float32))
    with pytest.raises(ValueError):
        mfe.MfeTensor((8, 16, 64), m.pools[:2])


def test_sharded_store(tmp_path):
    a = {"a": np.arange(3, dtype=np.float32)}
    b = {"b": np.arange(5, dtype=np.int32)}
    container.save(tmp_path / "m-00001-of-00002.mfq", F.FileHeader(model_arch="x"), a)
    container.save(tmp_path / "m-00002-of-00002.mfq", F.FileHeader(model_arch="x"), b)
    with F.open_mfq(tmp_path / "m-00002-of-00002.mfq") as store:
        assert sorted(store) == ["a", "b"] and store["b"].tolist() == [0, 1, 2, 3, 4]


def test_legacy_dtype_names():
    assert F.canonical_dtype("NINT4") == "NINT" and F.canonical_dtype("NVQ3J-L") == "NVQ"
    assert F.canonical_dtype("NINTM") == "MFE" and F.canonical_dtype("BF16") == "BF16"


def test_nint8_zero_roundtrip():
    import numpy as np
    from mfq_b200 import formats as F
    from mfq_b200.formats import nint8zero
    w = (np.random.default_rng(0).standard_normal((3, 8, 64)) * 0.1).astype(np.float32)
    t = nint8zero.quantize_nint8_zero(w, axis=1)
    back = nint8zero.unpack_nint8_zero(nint8zero.pack_nint8_zero(t))
    assert back.shape == (3, 8, 64) and back.axis == 1
    deq = F.dequantize(back)
    assert deq.shape == w.shape and np.abs(deq - w).max() <= np.abs(w).max() / 127 * 0.51 + 1e-4
