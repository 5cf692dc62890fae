"""GGUF import: container parsing, block decoders, name/config mapping, and the CLI path GGUF -> .mfq."""

import json

import numpy as np
import pytest

from mfq_b200.formats import gguf


def _tiny_llama(tmp_path, kind=gguf.GGML_F16):
    rng = np.random.default_rng(0)
    h, heads, kv, d, inter, vocab, layers = 64, 4, 2, 16, 128, 96, 2
    md = {"general.architecture": "llama", "general.name": "tiny", "llama.block_count": layers, "llama.embedding_length": h,
          "llama.feed_forward_length": inter, "llama.attention.head_count": heads, "llama.attention.head_count_kv": kv,
          "llama.rope.freq_base": 10000.0, "llama.attention.layer_norm_rms_epsilon": 1e-5,
          "tokenizer.ggml.tokens": [f"t{i}" for i in range(vocab)]}
    t = {"token_embd.weight": (rng.standard_normal((vocab, h)).astype(np.float32), kind),
         "output_norm.weight": (np.ones(h, np.float32), gguf.GGML_F32)}
    for i in range(layers):
        b = f"blk.{i}."
        t[b + "attn_norm.weight"] = (np.ones(h, np.float32), gguf.GGML_F32)
        t[b + "ffn_norm.weight"] = (np.ones(h, np.float32), gguf.GGML_F32)
        t[b + "attn_q.weight"] = (rng.standard_normal((heads * d, h)).astype(np.float32), kind)
        t[b + "attn_k.weight"] = (rng.standard_normal((kv * d, h)).astype(np.float32), kind)
        t[b + "attn_v.weight"] = (rng.standard_normal((kv * d, h)).astype(np.float32), kind)
        t[b + "attn_output.weight"] = (rng.standard_normal((h, heads * d)).astype(np.float32), kind)
        t[b + "ffn_gate.weight"] = (rng.standard_normal((inter, h)).astype(np.float32), kind)
        t[b + "ffn_up.weight"] = (rng.standard_normal((inter, h)).astype(np.float32), kind)
        t[b + "ffn_down.weight"] = (rng.standard_normal((h, inter)).astype(np.float32), kind)
    t["rope_freqs.weight"] = (np.ones(d // 2, np.float32), gguf.GGML_F32)  # no canonical name
    path = tmp_path / "tiny.gguf"
    gguf.write_gguf(path, md, t)
    return path, t, dict(h=h, heads=heads, kv=kv, d=d, inter=inter, vocab=vocab, layers=layers)


@pytest.mark.parametrize("kind,tol", [(gguf.GGML_F32, 0.0), (gguf.GGML_F16, 2e-3), (gguf.GGML_BF16, 1.6e-2),
                                      (gguf.GGML_Q8_0, 2e-2), (gguf.GGML_Q4_0, 0.3)])
def test_tensor_round_trip(tmp_path, kind, tol):
    x = np.random.default_rng(1).standard_normal((8, 64)).astype(np.float32)
    p = tmp_path / "t.gguf"
    gguf.write_gguf(p, {"general.architecture": "llama"}, {"a.weight": (x, kind), "b": (x[0], gguf.GGML_F32)})
    g = gguf.GgufFile(p)
    assert g.tensors["a.weight"].shape == (8, 64) and g.tensors["b"].shape == (64,)
    got = g.read("a.weight")
    assert np.abs(got - x).max() <= tol * max(1.0, np.abs(x).max())
    assert np.array_equal(g.read("b"), x[0])


def test_block_decoders_against_hand_built_blocks():
    # Q4_1: value = q * d + m; Q5_0: 5-bit q with the fifth bits in a u32, value = (q - 16) * d
    d, m = np.float16(0.5), np.float16(-1.0)
    nib = np.arange(16, dtype=np.uint8) | (np.arange(16, dtype=np.uint8)[::-1] << 4)
    q41 = np.frombuffer(d.tobytes() + m.tobytes() + nib.tobytes(), dtype=np.uint8)
    got = gguf.decode(q41, 0, 32, gguf.GGML_Q4_1)
    want = np.concatenate([np.arange(16), np.arange(16)[::-1]]).astype(np.float32) * 0.5 - 1.0
    assert np.array_equal(got, want)
    qh = np.uint32(0b1010).tobytes()  # values 1 and 3 get +16
    q50 = np.frombuffer(d.tobytes() + qh + nib.tobytes(), dtype=np.uint8)
    got = gguf.decode(q50, 0, 32, gguf.GGML_Q5_0)
    q = np.concatenate([np.arange(16), np.arange(16)[::-1]]).astype(np.float32)
    q[1] += 16
    q[3] += 16
    assert np.array_equal(got, (q - 16) * 0.5)


def test_llama_names_config_and_rope_permutation(tmp_path):
    path, t, dims = _tiny_llama(tmp_path, gguf.GGML_F32)
    cfg, tensors, assets = gguf.read_gguf(path)
    assert cfg["vocab_size"] == dims["vocab"] and cfg["num_layers"] == 2 and cfg["num_kv_heads"] == 2 and cfg["head_dim"] == 16
    assert "model.block.1.mlp.down.weight" in tensors and "model.output.weight" in tensors  # tied head filled in
    assert json.loads(assets["gguf_skipped.json"]) == ["rope_freqs.weight"]
    # the converter's interleaving of rotary pairs is undone: row 2i of a stored head is row i of its first half
    stored = t["blk.0.attn_q.weight"][0]
    got = tensors["model.block.0.attention.query.weight"]
    d = dims["d"]
    assert np.array_equal(got[0], stored[0]) and np.array_equal(got[1], stored[2]) and np.array_equal(got[d // 2], stored[1])
    assert np.array_equal(tensors["model.block.0.attention.value.weight"], t["blk.0.attn_v.weight"][0])


def test_cli_quantizes_a_gguf_file(tmp_path):
    from mfq_b200 import formats as F
    from mfq_b200.cli import main
    path, _, dims = _tiny_llama(tmp_path, gguf.GGML_Q8_0)
    out = tmp_path / "tiny.mfq"
    assert main(["quantize", str(path), str(out), "--bits", "4"]) == 0
    with F.open_mfq(out) as store:
        cfg = json.loads(store.assets()["model_config.json"])
        assert cfg["hidden_size"] == dims["h"] and "gguf_metadata.json" in store.assets()
        assert "model.block.0.attention.query.weight" in list(store)
