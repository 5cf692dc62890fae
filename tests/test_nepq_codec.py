"""NEPQ (cross-expert pooled tables, rotation, sparse residual): layout, round trip, formula by hand, encoder behaviour,
container / MFE integration, byte and value equality with the reference package."""

import struct

import numpy as np
import pytest

from mfq_b200 import formats as F
from mfq_b200.formats import nepq, npq0, nvq1


def _experts(e=3, out=8, k=136, seed=1):
    # 136 = five whole groups of 24 + a short one of 16: two super-groups, the second with two groups
    return (np.random.default_rng(seed).normal(size=(e, out, k)) * 0.05).astype(np.float32)


def _rel(t, w):
    rec = nepq.dequantize_nepq(t)
    return float(((rec - w) ** 2).sum() / (w ** 2).sum())


@pytest.mark.parametrize("name", list(nepq.PROFILES))
def test_layout_round_trip_and_error(name, tmp_path):
    w = _experts()
    t = nepq.quantize_nepq(w, name, banks=3)
    p = t.profile
    blob = nepq.pack_nepq(t)
    magic, ver, pid, per_super, flags, e, o, k, banks, block, seed = struct.unpack_from("<4sBBBBIIIIIQ", blob)
    assert (magic, ver, pid, per_super, e, o, k, banks) == (b"NEP1", 1, p.profile_id, 4, 3, 8, 136, 3)
    assert flags == (1 if block else 0) and bool(block) == bool(p.residual_block) and (not block or 136 % block == 0)
    ng, nv, ns = p.geometry(136)
    assert (ng, nv, ns) == (6, 17, 2) and t.state.shape == (3, 8, 6) and t.indices.shape == (3, 8, 17) and t.bank_ids.shape == (3, 8, 2)
    plain = 36 + p.stream_nbytes(24, 136, 3)
    if not p.residual_block:
        assert len(blob) == plain
    else:
        bpr = t.blocks_per_row
        assert bpr == -(-17 // p.residual_block) and blob[plain : plain + 4] == b"NRA1"
        extra = 64 + 1024 * 8 * 2 + (24 * bpr * p.record_bits + 7) // 8
        if p.residual_second:
            n2 = int(t.residual.second_mask.sum())
            extra += (24 * bpr + 7) // 8 + (n2 * p.record_bits + 7) // 8
            assert n2 == t.residual.second_records.size
        assert len(blob) == plain + extra
    back = nepq.unpack_nepq(blob)
    assert nepq.pack_nepq(back) == blob and np.array_equal(nepq.dequantize_nepq(back), nepq.dequantize_nepq(t))
    limit = {"NEPQ0-S": 0.50, "NEPQ0-L": 0.42, "NEPQ1-S": 0.27, "NEPQ1-L": 0.27, "NEPQ0-A": 0.46, "NEPQ1-A": 0.22}[name]
    assert _rel(t, w) < limit, _rel(t, w)
    path = tmp_path / "m.mfq"
    F.save(path, F.FileHeader(model_arch="test"), {"model.block.0.mlp.experts.down.weight": t})
    with F.open_mfq(path) as store:
        assert store.dtype("model.block.0.mlp.experts.down.weight") == "NEPQ"
        assert np.array_equal(F.dequantize(store["model.block.0.mlp.experts.down.weight"]), nepq.dequantize_nepq(t))


def test_reconstruction_formulas_by_hand():
    w = _experts(seed=2)
    t = nepq.quantize_nepq(w, "NEPQ0-L", banks=2)
    rec = nepq.dequantize_nepq(t)
    e, r, vec = 1, 5, 13  # vector 13 lies in group 4 = super-group 1
    bank = int(t.bank_ids[e, r, 1])
    ladder, first, second = npq0.unpack_tables(npq0.NPQ0_L, t.banks[bank].tobytes())
    s, i = int(t.state[e, r, 4]), int(t.indices[e, r, vec])
    want = t.anchors[e, r] * ladder[s] * np.concatenate([first[s, i & 7], second[s, i >> 3]]).astype(np.float32)
    assert np.allclose(rec[e, r, 104:112], want)
    t = nepq.quantize_nepq(w, "NEPQ1-S", banks=2)
    rec = nepq.dequantize_nepq(t)
    bank = int(t.bank_ids[e, r, 1])
    raw = t.banks[bank].tobytes()
    tables = np.stack([nvq1._unpack_table(raw[:1024], 512), nvq1._unpack_table(raw[1024:], 512)])
    a, q, i = int(t.aux[e, r, 4]), int(t.state[e, r, 4]), int(t.indices[e, r, vec])
    want = t.anchors[e, r] * q * (tables[a, i] + (-0.15625 if a else 0.15625))
    assert np.allclose(rec[e, r, 104:112], want)
    t = nepq.quantize_nepq(w, "NEPQ1-L", banks=2)
    assert np.array_equal(nvq1._unpack_table(t.banks[0].tobytes(), 2048), nvq1.IQ1S_GRID)  # bank 0 of the L pool is the grid


def test_rotation_is_orthonormal_and_undone():
    x = np.random.default_rng(3).normal(size=(5, 128)).astype(np.float32)
    y = nepq.rotate_rows(x, 32, seed=7)
    assert np.allclose((y ** 2).sum(1), (x ** 2).sum(1), rtol=1e-5) and np.allclose(nepq.unrotate_rows(y, 32, 7), x, atol=1e-6)
    h4 = nepq.hadamard_blocks(np.eye(4, dtype=np.float32), 4) * 2
    assert np.array_equal(h4, np.array([[1, 1, 1, 1], [1, -1, 1, -1], [1, 1, -1, -1], [1, -1, -1, 1]], dtype=np.float32))
    s = nepq.rotation_signs(128, 32, 7)
    assert s.dtype == np.int8 and set(np.unique(s).tolist()) == {-1, 1} and np.array_equal(s, nepq.rotation_signs(128, 32, 7))
    assert not np.array_equal(s, nepq.rotation_signs(128, 32, 8)) and not np.array_equal(s, nepq.rotation_signs(128, 64, 7))
    # outliers: a rotation spreads them over the block, which a coarse codec rewards
    w = _experts(e=2, out=16, k=128, seed=4)
    w[:, :, 5] *= 12.0
    plain = nepq.quantize_nepq(w, "NEPQ1-S", banks=2, rotation_block=0)
    turned = nepq.quantize_nepq(w, "NEPQ1-S", banks=2, rotation_block=64, rotation_seed=3)
    assert turned.rotation_block == 64 and _rel(turned, w) < _rel(plain, w)
    stored = nepq.dequantize_nepq(turned, logical=False)
    assert np.allclose(nepq.unrotate_rows(stored, 64, 3), nepq.dequantize_nepq(turned), atol=1e-6)


def test_residual_and_pool_behaviour():
    w = _experts(e=4, out=16, k=192, seed=5)
    base = nepq.quantize_nepq(w, "NEPQ1-S", banks=2, rotation_block=64)
    more = nepq.quantize_nepq(w, "NEPQ1-A", banks=2, rotation_block=64, pool=base.banks)
    assert np.array_equal(more.banks, base.banks) and _rel(more, w) < 0.9 * _rel(base, w)
    # the share of blocks with a second record follows the knob; none at 0
    none = nepq.quantize_nepq(w, "NEPQ1-A", banks=2, rotation_block=64, pool=base.banks, second_fraction=0.0)
    assert int(none.residual.second_mask.sum()) == 0 and none.residual.second_records.size == 0
    assert _rel(more, w) < _rel(none, w) < _rel(base, w)
    assert 0.4 <= more.residual.second_mask.mean() <= 0.5
    offsets, rows, ids = nepq.residual_by_vector(more)
    assert offsets.shape == (25,) and offsets[-1] == rows.size == ids.size == more.residual.first.size + more.residual.second_records.size
    # a frozen pool from other data still encodes; a bigger pool is never worse on the data it was trained on
    other = nepq.quantize_nepq(_experts(e=4, out=16, k=192, seed=6), "NEPQ0-S", banks=2)
    reuse = nepq.quantize_nepq(w, "NEPQ0-S", pool=other.banks)
    own1 = nepq.quantize_nepq(w, "NEPQ0-S", banks=1)
    own4 = nepq.quantize_nepq(w, "NEPQ0-S", banks=4)
    assert np.array_equal(reuse.banks, other.banks) and _rel(own4, w) <= _rel(own1, w) * 1.02
    assert len(set(np.unique(own4.bank_ids).tolist())) > 1  # the super-groups really spread over the banks
    with pytest.raises(ValueError):
        nepq.quantize_nepq(w, "NEPQ0-A", rotation_block=0)


def test_refusals():
    w = _experts()
    t = nepq.quantize_nepq(w, "NEPQ0-A", banks=2)
    blob = bytearray(nepq.pack_nepq(t))
    for edit in (lambda b: b.__setitem__(0, 0x58), lambda b: b.__setitem__(4, 2), lambda b: b.__setitem__(6, 8),
                 lambda b: b.__setitem__(7, 0), lambda b: b.append(0)):
        bad = bytearray(blob)
        edit(bad)
        with pytest.raises(ValueError):
            nepq.unpack_nepq(bytes(bad))
    with pytest.raises(ValueError):
        nepq.unpack_nepq(bytes(blob[:-3]))
    bad = nepq.NepqTensor(**{**t.__dict__, "bank_ids": t.bank_ids + 2})
    with pytest.raises(ValueError):
        nepq.pack_nepq(bad)
    pos = t.residual.first.copy()
    pos[0, 0, 0] = (5 << 5) | 30  # position 30 in a block of 17 vectors
    with pytest.raises(ValueError):
        nepq.pack_nepq(nepq.NepqTensor(**{**t.__dict__, "residual": nepq.NepqResidual(t.residual.dictionary, pos)}))
    with pytest.raises(ValueError):
        nepq.quantize_nepq(w[:, :, :100], "NEPQ0-S")
    with pytest.raises(ValueError):
        nepq.profile_of("NEPQ9")


def test_expert_mix_pools_share_one_table_pool_and_carry_the_rotation_record():
    from mfq_b200.formats.mfe import MfePool, MfeTensor, rotation_runtime
    from mfq_b200.quantize.expertwise import parse_profiles, quantize_expertwise
    w = _experts(e=4, out=8, k=96, seed=8)
    profiles = parse_profiles("NEPQ1-S,NINT4")
    mfe = quantize_expertwise(w, np.array([0, 1, 0, 0]), profiles)
    pool = next(p for p in mfe.pools if isinstance(p.tensor, nepq.NepqTensor))
    assert pool.tensor.shape == (3, 8, 96) and list(pool.expert_ids) == [0, 2, 3]
    rec = F.dequantize(mfe)
    assert rec.shape == w.shape and float(((rec - w) ** 2).sum() / (w ** 2).sum()) < 0.25
    rot = nepq.quantize_nepq(w, "NEPQ0-A", banks=1)
    packed = F.pack_tensor(MfeTensor(w.shape, (MfePool(np.arange(4, dtype=np.int32), rot),)))
    back = F.unpack_tensor(*packed)
    rt = back.pools[0].runtime
    assert rt == rotation_runtime(rot) and rt[:4] == b"HSG1" and struct.unpack_from("<4sIIQ", rt)[1:] == (96, rot.rotation_block, 0)
    assert np.array_equal(np.frombuffer(rt, dtype=np.int8, offset=20), nepq.rotation_signs(96, rot.rotation_block, 0))
    assert np.array_equal(F.dequantize(back), nepq.dequantize_nepq(rot))


def test_bytes_and_values_equal_the_reference_package(reference_pkg):
    from mfq.formats import nepq as R  # type: ignore
    w = _experts()
    for name in nepq.PROFILES:
        t = nepq.quantize_nepq(w, name, banks=3)
        blob = nepq.pack_nepq(t)
        theirs = R.unpack_nepq(blob)
        assert R.pack_nepq(theirs) == blob, name
        assert np.array_equal(R.dequantize_nepq(theirs), nepq.dequantize_nepq(t, logical=False)), name
        assert theirs.spec.label == name and theirs.payload_nbytes == len(blob) - 36
        if t.rotation_block:
            assert np.array_equal(R.rotation_signs(136, t.rotation_block, 0), nepq.rotation_signs(136, t.rotation_block, 0))
        if t.residual is not None:
            p, bpr = t.profile, t.blocks_per_row
            first = np.asarray(t.residual.first).reshape(-1, bpr).astype(np.int32)
            second = np.full_like(first, -1)
            if p.residual_second:
                flat = second.reshape(-1)
                flat[np.flatnonzero(t.residual.second_mask.reshape(-1))] = t.residual.second_records
            want = R.transpose_sparse_residual_records(first, second, vectors=17, block_vectors=p.residual_block, position_bits=p.position_bits)
            got = nepq.residual_by_vector(t)
            assert all(np.array_equal(a, b) for a, b in zip(want, got))


def test_checkpoint_with_pooled_experts_loads_and_serves(tmp_path, capsys):
    """`mfq quantize --random-expert-mix NEPQ1-S,NINT4`: the routed experts of a projection that drew NEPQ share one
    table pool inside their MFE record; the checkpoint evaluates against its source and loads into the engine."""
    import json

    import torch
    from mfq_b200.checkpoint import load_engine
    from mfq_b200.cli import main
    base, mixed = tmp_path / "base.mfq", tmp_path / "nepq.mfq"
    assert main(["quantize", "synthetic:tiny-moe-128", str(base), "--full-precision"]) == 0
    assert main(["quantize", "synthetic:tiny-moe-128", str(mixed), "--format", "nint4", "--random-expert-mix", "NEPQ1-S,NINT4"]) == 0
    with F.open_mfq(mixed) as store:
        name = next(n for n in store if n.endswith("mlp.experts.down.weight"))
        mfe = store[name]
        pooled = [p for p in mfe.pools if isinstance(p.tensor, nepq.NepqTensor)]
        assert store.dtype(name) == "MFE" and len(pooled) == 1 and pooled[0].tensor.shape[0] == len(pooled[0].expert_ids) == 4
    capsys.readouterr()
    assert main(["eval", "kl", "--model", str(mixed), "--base", str(base), "--chunks", "2", "--ctx", "64"]) == 0
    line = capsys.readouterr().out.strip()
    assert float(line.split()[0].split("=")[1]) < 0.05, line
    engine, tok, cfg = load_engine(mixed, "cpu", max_batch=2, max_seq_len=64)
    assert engine.generate([torch.tensor(tok.encode("hello"))], 4).tokens.shape == (1, 4)
