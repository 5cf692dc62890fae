"""Super-block GGUF tensor types (Q2_K .. Q6_K, IQ4_NL, IQ4_XS) against the `gguf` package's own dequantizers on random
block bytes, and through the file reader."""

import numpy as np
import pytest

from mfq_b200.formats import gguf as G

gguf_pkg = pytest.importorskip("gguf")

CASES = [("Q2_K", G.GGML_Q2_K, 84, 256, [80, 82]), ("Q3_K", G.GGML_Q3_K, 110, 256, [108]), ("Q4_K", G.GGML_Q4_K, 144, 256, [0, 2]),
         ("Q5_K", G.GGML_Q5_K, 176, 256, [0, 2]), ("Q6_K", G.GGML_Q6_K, 210, 256, [208]), ("IQ4_NL", G.GGML_IQ4_NL, 18, 32, [0]),
         ("IQ4_XS", G.GGML_IQ4_XS, 136, 256, [0])]


def _random_blocks(name, block_bytes, halves, count, seed):
    rng = np.random.default_rng(seed)
    raw = rng.integers(0, 256, size=(count, block_bytes), dtype=np.uint8)
    for off in halves:  # the fp16 multipliers must be finite numbers
        raw[:, off : off + 2] = np.frombuffer(rng.uniform(0.01, 0.1, count).astype("<f2").tobytes(), dtype=np.uint8).reshape(count, 2)
    return raw


@pytest.mark.parametrize("name,kind,block_bytes,values,halves", CASES)
def test_decode_equals_the_gguf_package(name, kind, block_bytes, values, halves):
    from gguf.quants import dequantize
    raw = _random_blocks(name, block_bytes, halves, 9, seed=values + block_bytes)
    want = dequantize(raw.reshape(-1), getattr(gguf_pkg.GGMLQuantizationType, name)).reshape(-1)
    got = G.decode(raw.reshape(-1), 0, 9 * values, kind)
    assert got.dtype == np.float32 and np.array_equal(got, want.astype(np.float32))


def test_reader_sizes_a_super_block_tensor(tmp_path):
    """A file holding one Q4_K matrix followed by an F32 vector: the second tensor's offset proves the first one's size."""
    from gguf.quants import dequantize
    rows, cols = 4, 512
    raw = _random_blocks("Q4_K", 144, [0, 2], rows * cols // 256, seed=3)
    vec = np.arange(8, dtype=np.float32)
    path = tmp_path / "k.gguf"
    name_a, name_b = b"blk.0.ffn_down.weight", b"output_norm.weight"
    head = G.MAGIC + np.array([3], "<u4").tobytes() + np.array([2, 0], "<u8").tobytes()
    off_b = (raw.size + 31) // 32 * 32
    info = b""
    for nm, dims, kind, off in ((name_a, (cols, rows), G.GGML_Q4_K, 0), (name_b, (8,), G.GGML_F32, off_b)):
        info += np.array([len(nm)], "<u8").tobytes() + nm + np.array([len(dims)], "<u4").tobytes()
        info += np.array(dims, "<u8").tobytes() + np.array([kind], "<u4").tobytes() + np.array([off], "<u8").tobytes()
    body = head + info
    pad = (-len(body)) % 32
    data = raw.tobytes() + b"\0" * (off_b - raw.size) + vec.tobytes()
    path.write_bytes(body + b"\0" * pad + data)
    f = G.GgufFile(path)
    want = dequantize(raw.reshape(-1), gguf_pkg.GGMLQuantizationType.Q4_K).reshape(rows, cols)
    assert np.array_equal(f.read("blk.0.ffn_down.weight"), want.astype(np.float32))
    assert np.array_equal(f.read("output_norm.weight"), vec)
