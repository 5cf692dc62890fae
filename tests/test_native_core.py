"""Host runtime library (C++): container reader, NINT row decoder, prefix cache, planners -- against the Python twins."""

import hashlib

import numpy as np
import pytest

from mfq_b200 import formats as F
from mfq_b200 import native
from mfq_b200.formats import container, nint
from mfq_b200.quantize.nint import quantize_nint


def _nint_tensor(rows, cols, seed, bits=4):
    w = np.random.default_rng(seed).standard_normal((rows, cols)).astype(np.float32)
    return quantize_nint(w, nint.NintSpec(bits=bits, groupsize=32, sub_bits=6))


def test_store_matches_python_reader(tmp_path):
    t1, t2 = _nint_tensor(24, 96, 0), np.arange(40, dtype=np.float32).reshape(5, 8)
    path = tmp_path / "m.mfq"
    container.save(path, container.FileHeader(model_arch="llama", extra={"k": {"a": 1}}),
                   {"model.a.weight": t1, "model.b.weight": t2, "__mfq_asset__/x.json": b"{}"})
    py = container.open_mfq(path)
    with native.NativeStore(path) as st:
        assert st.arch == "llama" and st.extra == {"k": '{"a": 1}'} and len(st) == 3
        assert st.names == list(py)
        for i, name in enumerate(st.names):
            rec = py.records[name]
            assert st.info(i)[1:3] == (rec.dtype, rec.nbytes) and st.find(name) == i
            raw = bytes(st.view(i))
            assert raw == bytes(py.raw(name))
            buf = np.empty(len(raw), dtype=np.uint8)
            st.read_into(i, buf, threads=3)
            assert buf.tobytes() == raw
        assert st.find("missing") == -1


def test_sharded_store(tmp_path):
    tensors = {f"model.block.{i}.w": np.full((4, 4), i, dtype=np.float32) for i in range(5)}
    names = list(tensors)
    paths = [tmp_path / f"s-{i + 1:05d}-of-00003.mfq" for i in range(3)]
    for i, path in enumerate(paths):
        container.save(path, container.FileHeader(model_arch="x"), {n: tensors[n] for n in names[2 * i : 2 * i + 2]})
    with native.NativeStore(paths[1]) as st:  # any shard opens the whole set
        assert sorted(st.names) == sorted(tensors) and {st.info(i)[3] for i in range(len(st))} == {0, 1, 2}


@pytest.mark.parametrize("bits,rows,cols", [(4, 24, 96), (3, 17, 160), (6, 5, 70)])
def test_nint_rows_decode_and_gemv(bits, rows, cols):
    t = _nint_tensor(rows, cols, bits, bits=bits)
    # mix per-row widths so that every selector class path is exercised
    t.row_q_bits = np.full(rows, bits, dtype=np.uint8)
    t.row_sub_bits = np.full(rows, 6, dtype=np.uint8)
    t.row_q_bits[::3] = max(1, bits - 1)
    t.row_sub_bits[1::4] = 7
    t.q[::3] = np.minimum(t.q[::3], (1 << max(1, bits - 1)) - 1)
    blob = np.frombuffer(nint.pack_nint(t), dtype=np.uint8)
    want = nint.dequantize_nint_rows(nint.unpack_nint(blob.tobytes()))
    dec = native.NintRows(blob)
    assert (dec.rows, dec.row_len) == (rows, cols)
    np.testing.assert_allclose(dec.decode(threads=4), want, rtol=1e-6, atol=1e-7)
    np.testing.assert_allclose(dec.decode(1, min(rows, 9)), want[1:9], rtol=1e-6, atol=1e-7)
    x = np.random.default_rng(1).standard_normal(cols).astype(np.float32)
    np.testing.assert_allclose(dec.gemv(x), want @ x, rtol=1e-4, atol=1e-4)
    assert dec.row_bits(0)[0] == int(t.row_q_bits[0])


def test_mx_and_fp8_decoders():
    rng = np.random.default_rng(0)
    w = rng.standard_normal((8, 64)).astype(np.float32)
    from mfq_b200.quantize.mxfp4 import quantize_mxfp4
    t = quantize_mxfp4(w)
    np.testing.assert_array_equal(native.mxfp4_decode(t.values, t.scales, 8, 64), F.dequantize(t))
    codes = rng.integers(0, 256, (130, 140), dtype=np.uint8)
    codes[(codes & 0x7F) == 0x7F] = 0
    scales = rng.random((2, 2), dtype=np.float32)
    from mfq_b200.formats.mx import e4m3_to_float
    want = e4m3_to_float(codes) * np.repeat(np.repeat(scales, 128, 0), 128, 1)[:130, :140]
    np.testing.assert_allclose(native.fp8_block_decode(codes, scales), want, rtol=1e-6)


def test_prefix_cache_keys_tiers_and_pins(tmp_path):
    pc = native.PrefixCache(tmp_path / "kv", ram_budget=3000, disk_budget=10_000, block_tokens=4)
    toks = np.arange(14, dtype=np.int32)
    keys = pc.keys(toks, salt="m1")
    assert keys.shape == (3, 32)
    prev = bytes(32)
    for b in range(3):  # the chain is plain SHA-256, so any implementation can recompute it
        prev = hashlib.sha256(prev + toks[4 * b : 4 * b + 4].tobytes() + b"m1").digest()
        assert keys[b].tobytes() == prev
    assert not np.array_equal(pc.keys(toks, salt="m2")[0], keys[0])
    other = toks.copy()
    other[5] = 99  # a change in block 1 leaves key 0 alone and changes every later key
    k2 = pc.keys(other, salt="m1")
    assert np.array_equal(k2[0], keys[0]) and not np.array_equal(k2[1], keys[1]) and not np.array_equal(k2[2], keys[2])
    blocks = [np.full(1000, i, dtype=np.uint8) for i in range(3)]
    for k, b in zip(keys, blocks):
        pc.put(k, b)
    pc.flush()
    assert pc.match(keys) == 3 and pc.match(k2) == 1
    st = pc.stats()
    assert st["ram_bytes"] <= 3000 and st["disk_entries"] == 3
    for k, b in zip(keys, blocks):
        np.testing.assert_array_equal(pc.get(k, 1000), b)
    assert pc.get(k2[2], 1000) is None
    st = pc.stats()
    assert st["hits_ram"] + st["hits_disk"] == 3 and st["misses"] == 1
    pc.close()
    # a new process adopts the file tier
    pc2 = native.PrefixCache(tmp_path / "kv", ram_budget=3000, disk_budget=10_000, block_tokens=4)
    assert pc2.match(keys) == 3
    np.testing.assert_array_equal(pc2.get(keys[1], 1000), blocks[1])
    pc2.close()
    # RAM-only cache: pinned entries survive eviction pressure
    pc3 = native.PrefixCache(None, ram_budget=2000, block_tokens=4)
    pc3.put(keys[0], blocks[0])
    pc3.pin(keys[0])
    pc3.put(keys[1], blocks[1])
    pc3.put(keys[2], blocks[2])
    assert pc3.get(keys[0], 1000) is not None and pc3.stats()["ram_bytes"] <= 2000 + 1000
    pc3.close()


def test_planners():
    assert native.tp_plan(1024, 8, granularity=128) == [(i * 128, (i + 1) * 128) for i in range(8)]
    plan = native.tp_plan(1280, 3, weights=[2, 1, 1], granularity=128)
    assert plan[0][0] == 0 and plan[-1][1] == 1280 and all(b % 128 == 0 and e % 128 == 0 for b, e in plan)
    assert [e - b for b, e in plan] == [640, 384, 256] or [e - b for b, e in plan] == [640, 256, 384]
    with pytest.raises(ValueError):
        native.tp_plan(100, 2, granularity=64)
    heat = [5.0, 0.1, 3.0, 9.0, 0.2, 7.0]
    resident = [1, 1, 1, 0, 0, 0]
    assert native.moe_rank_swaps(heat, resident, 4) == [(1, 3), (2, 5)]
    assert native.moe_rank_swaps(heat, resident, 1) == [(1, 3)]
    tiers = native.moe_dispatch_plan([0, 4, 1, 4000], [1, 1, 0, 0], bytes_per_expert=50e6, h2d_gbs=50, gpu_tok_us=0.05, cpu_tok_us=20)
    assert tiers.tolist() == [native.TIER_INACTIVE, native.TIER_GPU_RESIDENT, native.TIER_CPU, native.TIER_GPU_TRANSFER]
    book = native.SlotBook(2)
    assert book.acquire(10) == (1, None) or book.acquire(10)[1] is None
    s10 = book.lookup(10)
    s11, _ = book.acquire(11)
    assert {s10, s11} == {0, 1}
    book.pin(11)
    book.lookup(10)
    slot, evicted = book.acquire(12)  # 11 is pinned, so 10 goes although it is more recent
    assert evicted == 10 and slot == s10 and book.lookup(10) == -1
    book.pin(12)
    with pytest.raises(MemoryError):
        book.acquire(13)


def test_native_nvq_rows_match_the_python_decoder():
    import numpy as np
    from mfq_b200 import formats as F
    from mfq_b200 import native
    from mfq_b200.formats.nvq import dequantize_nvq_rows
    from mfq_b200.quantize.nvq import quantize_nvq
    rng = np.random.default_rng(0)
    for cb, cols in (("e8_1024", 200), ("d4_512", 96), ("e8_256", 72)):
        w = rng.standard_normal((12, cols)).astype(np.float32)
        t = quantize_nvq(w, F.NvqSpec(cb))
        got = native.nvq_decode(t, threads=3)
        assert got.shape == (12, cols) and np.array_equal(got, dequantize_nvq_rows(t).astype(np.float32))
    t.indices = t.indices.astype(np.uint16)
    t.indices[0, 0] = 60000
    import pytest
    with pytest.raises(ValueError):
        native.nvq_decode(t)
