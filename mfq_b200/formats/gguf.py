"""GGUF import: read a llama.cpp ``.gguf`` file (metadata, tensor table, common ggml tensor encodings) and map it to
canonical tensor names and a model config, so ``mfq quantize model.gguf out.mfq`` works like it does for a Hugging
Face directory.  A small writer exists for tests and fixtures.

File layout (little endian): ``"GGUF"``, version u32 (2 or 3), tensor count u64, key/value count u64; the key/value
pairs (string key, u32 type, value; arrays carry an element type and a u64 count); the tensor infos (name, u32 rank,
u64 dims with the innermost first, u32 ggml type, u64 offset into the data section); padding to ``general.alignment``
(default 32); tensor data.  Decoded here: F32, F16, BF16, Q8_0, Q4_0, Q4_1, Q5_0, Q5_1 (blocks of 32), the 256-value super-block
types Q2_K .. Q6_K, IQ4_NL and IQ4_XS.  Reference:
``mfq/tools/quantize_gguf_to_mfq.py`` (the reference's GGUF front end) and ``mfq/commands/quantize.py:308-322``
(source detection).
"""

from __future__ import annotations

import json
import struct
from dataclasses import dataclass
from pathlib import Path

import numpy as np

MAGIC = b"GGUF"
_SCALARS = {0: "<B", 1: "<b", 2: "<H", 3: "<h", 4: "<I", 5: "<i", 6: "<f", 7: "<?", 10: "<Q", 11: "<q", 12: "<d"}
T_STRING, T_ARRAY = 8, 9
GGML_F32, GGML_F16, GGML_Q4_0, GGML_Q4_1, GGML_Q5_0, GGML_Q5_1, GGML_Q8_0, GGML_BF16 = 0, 1, 2, 3, 6, 7, 8, 30
_BLOCK_BYTES = {GGML_Q4_0: 18, GGML_Q4_1: 20, GGML_Q5_0: 22, GGML_Q5_1: 24, GGML_Q8_0: 34}


@dataclass
class TensorInfo:
    name: str
    shape: tuple[int, ...]  # outermost first (numpy order)
    ggml_type: int
    offset: int  # into the data section


class _Reader:
    def __init__(self, buf: memoryview) -> None:
        self.buf, self.pos = buf, 0

    def take(self, fmt: str):
        v = struct.unpack_from(fmt, self.buf, self.pos)
        self.pos += struct.calcsize(fmt)
        return v[0]

    def string(self) -> str:
        n = self.take("<Q")
        s = bytes(self.buf[self.pos : self.pos + n]).decode("utf-8", errors="replace")
        self.pos += n
        return s

    def value(self, kind: int):
        if kind in _SCALARS:
            return self.take(_SCALARS[kind])
        if kind == T_STRING:
            return self.string()
        if kind == T_ARRAY:
            elem, count = self.take("<I"), self.take("<Q")
            if elem in _SCALARS and elem != 7:
                dt = np.dtype(_SCALARS[elem])
                out = np.frombuffer(self.buf, dtype=dt, count=count, offset=self.pos)
                self.pos += count * dt.itemsize
                return out
            return [self.value(elem) for _ in range(count)]
        raise ValueError(f"unknown GGUF value type {kind}")


class GgufFile:
    """Memory-mapped GGUF file: ``metadata`` dict, ``tensors`` table, ``read(name)`` -> float32 array."""

    def __init__(self, path) -> None:
        self.path = Path(path)
        self._mm = np.memmap(self.path, dtype=np.uint8, mode="r")
        r = _Reader(memoryview(self._mm))
        if bytes(r.buf[:4]) != MAGIC:
            raise ValueError(f"{path}: not a GGUF file")
        r.pos = 4
        self.version = r.take("<I")
        if self.version not in (2, 3):
            raise ValueError(f"{path}: GGUF version {self.version} is not supported")
        n_tensors, n_kv = r.take("<Q"), r.take("<Q")
        self.metadata: dict[str, object] = {}
        for _ in range(n_kv):
            key = r.string()
            self.metadata[key] = r.value(r.take("<I"))
        self.tensors: dict[str, TensorInfo] = {}
        for _ in range(n_tensors):
            name = r.string()
            rank = r.take("<I")
            dims = [r.take("<Q") for _ in range(rank)]
            kind, off = r.take("<I"), r.take("<Q")
            self.tensors[name] = TensorInfo(name, tuple(reversed(dims)), kind, off)
        align = int(self.metadata.get("general.alignment", 32))
        self.data_start = (r.pos + align - 1) // align * align

    def read(self, name: str) -> np.ndarray:
        info = self.tensors[name]
        n = int(np.prod(info.shape)) if info.shape else 1
        start = self.data_start + info.offset
        return decode(self._mm, start, n, info.ggml_type).reshape(info.shape)


def _f16(raw: np.ndarray) -> np.ndarray:
    return raw.view("<f2").astype(np.float32)


def decode(buf: np.ndarray, start: int, n: int, kind: int) -> np.ndarray:
    """``n`` values of ggml type ``kind`` starting at byte ``start`` of ``buf`` as float32."""
    if kind == GGML_F32:
        return np.frombuffer(buf, dtype="<f4", count=n, offset=start).astype(np.float32)
    if kind == GGML_F16:
        return np.frombuffer(buf, dtype="<f2", count=n, offset=start).astype(np.float32)
    if kind == GGML_BF16:
        raw = np.frombuffer(buf, dtype="<u2", count=n, offset=start).astype(np.uint32) << 16
        return raw.view(np.float32)
    if kind in _SUPER_BLOCK_BYTES or kind == GGML_IQ4_NL:
        return _decode_k(buf, start, n, kind)
    if kind not in _BLOCK_BYTES:
        raise NotImplementedError(f"ggml tensor type {kind} is not decoded here (F32, F16, BF16, Q8_0, Q4_0/1, Q5_0/1, "
                                  "Q2_K .. Q6_K, IQ4_NL and IQ4_XS are)")
    if n % 32:
        raise ValueError("block-quantized tensors hold a multiple of 32 values")
    nb, bb = n // 32, _BLOCK_BYTES[kind]
    blocks = np.frombuffer(buf, dtype=np.uint8, count=nb * bb, offset=start).reshape(nb, bb)
    d = _f16(np.ascontiguousarray(blocks[:, :2]))
    if kind == GGML_Q8_0:
        q = blocks[:, 2:].view(np.int8).astype(np.float32)
        return (q * d).reshape(-1)
    has_min = kind in (GGML_Q4_1, GGML_Q5_1)
    pos = 2
    m = None
    if has_min:
        m = _f16(np.ascontiguousarray(blocks[:, 2:4]))
        pos = 4
    high = None
    if kind in (GGML_Q5_0, GGML_Q5_1):
        qh = np.ascontiguousarray(blocks[:, pos : pos + 4]).view("<u4")  # bit j = fifth bit of value j
        high = ((qh >> np.arange(32, dtype=np.uint32)) & 1).astype(np.uint8) << 4
        pos += 4
    nib = blocks[:, pos : pos + 16]
    q = np.concatenate([nib & 0x0F, nib >> 4], axis=1)  # values 0..15 are the low nibbles, 16..31 the high ones
    if high is not None:
        q = q | high
    q = q.astype(np.float32)
    if has_min:
        return (q * d + m).reshape(-1)
    return ((q - (16.0 if high is not None else 8.0)) * d).reshape(-1)


# ---- 256-value super-blocks (the "K" family) and the 4-bit non-linear types ---------------------------------------------
GGML_Q2_K, GGML_Q3_K, GGML_Q4_K, GGML_Q5_K, GGML_Q6_K, GGML_IQ4_NL, GGML_IQ4_XS = 10, 11, 12, 13, 14, 20, 23
_SUPER_BLOCK_BYTES = {GGML_Q2_K: 84, GGML_Q3_K: 110, GGML_Q4_K: 144, GGML_Q5_K: 176, GGML_Q6_K: 210, GGML_IQ4_XS: 136}
_IQ4_VALUES = np.array([-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113], dtype=np.float32)


def _scale_min_6bit(sc: np.ndarray) -> tuple[np.ndarray, np.ndarray]:
    """The eight 6-bit (scale, min) pairs packed in 12 bytes of a Q4_K / Q5_K block: ``[blocks, 8]`` each."""
    lo, mid, hi = sc[:, 0:4], sc[:, 4:8], sc[:, 8:12]
    scale = np.concatenate([lo & 63, (hi & 0x0F) | ((lo >> 6) << 4)], axis=1)
    mins = np.concatenate([mid & 63, (hi >> 4) | ((mid >> 6) << 4)], axis=1)
    return scale.astype(np.float32), mins.astype(np.float32)


def _decode_k(buf: np.ndarray, start: int, n: int, kind: int) -> np.ndarray:
    """Super-block types: every block of 256 values (32 for IQ4_NL) carries an fp16 multiplier and packed sub-block
    scales; the sub-block order below is the one ggml's reference dequantizers walk."""
    if kind == GGML_IQ4_NL:
        if n % 32:
            raise ValueError("IQ4_NL tensors hold a multiple of 32 values")
        blocks = np.frombuffer(buf, dtype=np.uint8, count=n // 32 * 18, offset=start).reshape(-1, 18)
        d = _f16(np.ascontiguousarray(blocks[:, :2]))
        nib = blocks[:, 2:]
        q = np.concatenate([nib & 0x0F, nib >> 4], axis=1)
        return (_IQ4_VALUES[q] * d).reshape(-1)
    if n % 256:
        raise ValueError("super-block tensors hold a multiple of 256 values")
    nb, bb = n // 256, _SUPER_BLOCK_BYTES[kind]
    blk = np.frombuffer(buf, dtype=np.uint8, count=nb * bb, offset=start).reshape(nb, bb)

    def f16(a, b):
        return _f16(np.ascontiguousarray(blk[:, a:b]))

    if kind == GGML_Q2_K:
        scales, qs, d, dmin = blk[:, :16], blk[:, 16:80], f16(80, 82), f16(82, 84)
        # value (half, shift j, l) reads byte qs[32 half + l], bits 2j..2j+1; its scale is number 8 half + 2 j + l // 16
        q = qs.reshape(nb, 2, 1, 32) >> (2 * np.arange(4, dtype=np.uint8)).reshape(1, 1, 4, 1) & 3
        sc = scales.reshape(nb, 2, 4, 2).repeat(16, axis=3)
        out = d[:, :, None, None] * (sc & 0x0F) * q - dmin[:, :, None, None] * (sc >> 4)
        return out.astype(np.float32).reshape(-1)
    if kind == GGML_Q3_K:
        hmask, qs, packed, d = blk[:, :32], blk[:, 32:96], blk[:, 96:108], f16(108, 110)
        aux = np.ascontiguousarray(packed).view("<u4").astype(np.uint32)  # [nb, 3]
        k1, k2 = np.uint32(0x03030303), np.uint32(0x0F0F0F0F)
        tmp = aux[:, 2]
        words = np.stack([(aux[:, 0] & k2) | ((tmp & k1) << 4), (aux[:, 1] & k2) | (((tmp >> 2) & k1) << 4),
                          ((aux[:, 0] >> 4) & k2) | (((tmp >> 4) & k1) << 4),
                          ((aux[:, 1] >> 4) & k2) | (((tmp >> 6) & k1) << 4)], axis=1).astype("<u4")
        sc = np.ascontiguousarray(words).view(np.uint8).reshape(nb, 16).astype(np.float32) - 32.0
        low = (qs.reshape(nb, 2, 1, 32) >> (2 * np.arange(4, dtype=np.uint8)).reshape(1, 1, 4, 1) & 3).astype(np.float32)
        bit = (hmask.reshape(nb, 1, 1, 32) >> np.arange(8, dtype=np.uint8).reshape(1, 2, 4, 1)) & 1  # bit 4 half + j
        q = low - np.where(bit == 1, 0.0, 4.0)
        out = d[:, :, None, None] * sc.reshape(nb, 2, 4, 2).repeat(16, axis=3) * q
        return out.astype(np.float32).reshape(-1)
    if kind in (GGML_Q4_K, GGML_Q5_K):
        d, dmin = f16(0, 2), f16(2, 4)
        scale, mins = _scale_min_6bit(blk[:, 4:16])
        if kind == GGML_Q4_K:
            ql = blk[:, 16:144].reshape(nb, 4, 32)
            high = np.zeros((nb, 4, 2, 32), dtype=np.uint8)
        else:
            qh, ql = blk[:, 16:48], blk[:, 48:176].reshape(nb, 4, 32)
            # values 64 j + l take bit 2 j of qh[l], values 64 j + 32 + l bit 2 j + 1
            high = ((qh.reshape(nb, 1, 1, 32) >> np.arange(8, dtype=np.uint8).reshape(1, 4, 2, 1)) & 1) << 4
        q = np.stack([ql & 0x0F, ql >> 4], axis=2) | high  # [nb, 4, 2, 32]
        out = (d * scale).reshape(nb, 4, 2, 1) * q - (dmin * mins).reshape(nb, 4, 2, 1)
        return out.astype(np.float32).reshape(-1)
    if kind == GGML_Q6_K:
        ql, qh = blk[:, :128].reshape(nb, 2, 2, 32), blk[:, 128:192].reshape(nb, 2, 1, 32)
        sc = blk[:, 192:208].view(np.int8).astype(np.float32).reshape(nb, 2, 4, 2)
        d = f16(208, 210)
        # per half: values l, l + 32 take the low nibbles of ql[l], ql[l + 32]; l + 64, l + 96 the high ones;
        # two more bits each come from qh[l] at shifts 0, 2, 4, 6
        nib = np.concatenate([ql & 0x0F, ql >> 4], axis=2)  # [nb, 2, 4, 32]
        top = (qh >> (2 * np.arange(4, dtype=np.uint8)).reshape(1, 1, 4, 1)) & 3
        q = (nib | (top << 4)).astype(np.float32) - 32.0
        out = d[:, :, None, None] * sc.repeat(16, axis=3) * q
        return out.astype(np.float32).reshape(-1)
    if kind == GGML_IQ4_XS:
        d = f16(0, 2)
        sh = np.ascontiguousarray(blk[:, 2:4]).view("<u2").astype(np.uint32)  # [nb, 1]
        sl, qs = blk[:, 4:8], blk[:, 8:136].reshape(nb, 8, 16)
        ib = np.arange(8)
        ls = ((sl[:, ib // 2] >> (4 * (ib % 2)).astype(np.uint8)) & 0x0F).astype(np.uint32) | (((sh >> (2 * ib).astype(np.uint32)) & 3) << 4)
        q = np.concatenate([qs & 0x0F, qs >> 4], axis=2)  # [nb, 8, 32]
        out = (d * (ls.astype(np.float32) - 32.0))[:, :, None] * _IQ4_VALUES[q]
        return out.astype(np.float32).reshape(-1)
    raise NotImplementedError(kind)


# ---- names and config -------------------------------------------------------------------------------------------
_BLOCK = {
    "attn_norm.weight": "attention.norm.weight", "attn_q.weight": "attention.query.weight", "attn_k.weight": "attention.key.weight",
    "attn_v.weight": "attention.value.weight", "attn_output.weight": "attention.output.weight",
    "attn_q_norm.weight": "attention.query_norm.weight", "attn_k_norm.weight": "attention.key_norm.weight",
    "ffn_norm.weight": "mlp.norm.weight", "ffn_gate.weight": "mlp.gate.weight", "ffn_up.weight": "mlp.up.weight",
    "ffn_down.weight": "mlp.down.weight", "ffn_gate_inp.weight": "mlp.router.weight",
    "ffn_gate_exps.weight": "mlp.experts.gate.weight", "ffn_up_exps.weight": "mlp.experts.up.weight",
    "ffn_down_exps.weight": "mlp.experts.down.weight", "ffn_gate_shexp.weight": "mlp.shared_expert.gate.weight",
    "ffn_up_shexp.weight": "mlp.shared_expert.up.weight", "ffn_down_shexp.weight": "mlp.shared_expert.down.weight",
    "ffn_gate_inp_shexp.weight": "mlp.shared_expert.router.weight", "ffn_gate_up_exps.weight": "mlp.experts.gate_up.weight",
    "post_attention_norm.weight": "mlp.norm.weight", "exp_probs_b.bias": "mlp.router.bias",
    # hybrid family (Gated DeltaNet layers), llama.cpp's names for them (mfq/architectures/tensor_schema.py:584-595)
    "attn_qkv.weight": "linear_attention.qkv.weight", "attn_gate.weight": "linear_attention.gate.weight",
    "ssm_alpha.weight": "linear_attention.alpha.weight", "ssm_beta.weight": "linear_attention.beta.weight",
    "ssm_conv1d.weight": "linear_attention.conv.weight", "ssm_dt.bias": "linear_attention.dt_bias",
    "ssm_a": "linear_attention.a", "ssm_norm.weight": "linear_attention.norm.weight", "ssm_out.weight": "linear_attention.output.weight",
    # latent attention (DeepSeek style)
    "attn_q_a.weight": "attention.query_a.weight", "attn_q_a_norm.weight": "attention.query_a_norm.weight",
    "attn_q_b.weight": "attention.query_b.weight", "attn_kv_a_mqa.weight": "attention.key_value_a.weight",
    "attn_kv_a_norm.weight": "attention.key_value_a_norm.weight", "attn_kv_b.weight": "attention.key_value_b.source.weight",
    # appended next-token-prediction layer
    "nextn.eh_proj.weight": "predictor.fusion.weight", "nextn.enorm.weight": "predictor.embedding_norm.weight",
    "nextn.hnorm.weight": "predictor.hidden_norm.weight", "nextn.shared_head_norm.weight": "predictor.output_norm.weight",
}
_TOP = {"token_embd.weight": "model.token_embedding.weight", "output_norm.weight": "model.output_norm.weight",
        "output.weight": "model.output.weight"}


def canonical_name(name: str) -> str | None:
    if name in _TOP:
        return _TOP[name]
    if name.startswith("blk."):
        _, idx, rest = name.split(".", 2)
        if rest in _BLOCK:
            target = _BLOCK[rest]
            return target if target.startswith("predictor.") else f"model.block.{idx}.{target}"
    return None


def _unpermute_rope(w: np.ndarray, heads: int) -> np.ndarray:
    """llama.cpp's converter stores q/k of the ``llama`` architecture with each head's rotary pairs interleaved;
    the rotate-half convention used here wants the two halves contiguous.  Inverse of that permutation."""
    rows = w.shape[0]
    return w.reshape(heads, rows // heads // 2, 2, *w.shape[1:]).swapaxes(1, 2).reshape(w.shape)


def config_from_metadata(md: dict, tensors: dict[str, TensorInfo]) -> dict:
    arch = str(md.get("general.architecture", "llama"))

    def get(key, default=None):
        return md.get(f"{arch}.{key}", default)

    heads = int(get("attention.head_count", 32))
    hidden = int(get("embedding_length"))
    vocab = len(md["tokenizer.ggml.tokens"]) if "tokenizer.ggml.tokens" in md else tensors["token_embd.weight"].shape[0]
    cfg = {"vocab_size": int(vocab), "hidden_size": hidden, "num_layers": int(get("block_count")), "num_heads": heads,
           "num_kv_heads": int(get("attention.head_count_kv", heads)), "head_dim": int(get("attention.key_length", hidden // heads)),
           "intermediate_size": int(get("feed_forward_length", 0)), "rope_theta": float(get("rope.freq_base", 1e4)),
           "rms_eps": float(get("attention.layer_norm_rms_epsilon", 1e-5)), "name": str(md.get("general.name", arch))}
    experts = int(get("expert_count", 0) or 0)
    if experts:
        cfg.update(num_experts=experts, top_k=int(get("expert_used_count", 2)),
                   moe_intermediate=int(get("expert_feed_forward_length", cfg["intermediate_size"])),
                   shared_intermediate=int(get("expert_shared_feed_forward_length", 0) or 0))
    return cfg


def read_gguf(path) -> tuple[dict, dict[str, np.ndarray], dict[str, bytes]]:
    """``.gguf`` -> (config, canonical float32 tensors, assets).  Tensors without a canonical name are reported in the
    ``gguf_skipped.json`` asset instead of being dropped silently."""
    g = GgufFile(path)
    cfg = config_from_metadata(g.metadata, g.tensors)
    arch = str(g.metadata.get("general.architecture", "llama"))
    out: dict[str, np.ndarray] = {}
    skipped = []
    for name in g.tensors:
        cname = canonical_name(name)
        if cname is None:
            skipped.append(name)
            continue
        w = g.read(name)
        if arch == "llama" and cname.endswith("attention.query.weight"):
            w = _unpermute_rope(w, cfg["num_heads"])
        if arch == "llama" and cname.endswith("attention.key.weight"):
            w = _unpermute_rope(w, cfg["num_kv_heads"])
        out[cname] = np.ascontiguousarray(w, dtype=np.float32)
    if "model.output.weight" not in out and "model.token_embedding.weight" in out:
        out["model.output.weight"] = out["model.token_embedding.weight"]  # tied embeddings
    assets = {"gguf_metadata.json": json.dumps({k: (v if isinstance(v, (int, float, str, bool)) else f"<{type(v).__name__}>")
                                                for k, v in g.metadata.items()}).encode()}
    if skipped:
        assets["gguf_skipped.json"] = json.dumps(skipped).encode()
    return cfg, out, assets


# ---- writer (fixtures) --------------------------------------------------------------------------------------------
def _pack_string(s: str) -> bytes:
    b = s.encode()
    return struct.pack("<Q", len(b)) + b


def _pack_value(v) -> bytes:
    if isinstance(v, bool):
        return struct.pack("<I?", 7, v)
    if isinstance(v, int):
        return struct.pack("<Iq", 11, v) if v < 0 else struct.pack("<II", 4, v) if v < 2 ** 32 else struct.pack("<IQ", 10, v)
    if isinstance(v, float):
        return struct.pack("<If", 6, v)
    if isinstance(v, str):
        return struct.pack("<I", T_STRING) + _pack_string(v)
    if isinstance(v, (list, tuple)) and all(isinstance(x, str) for x in v):
        return struct.pack("<IIQ", T_ARRAY, T_STRING, len(v)) + b"".join(_pack_string(x) for x in v)
    raise TypeError(f"cannot store {type(v).__name__} in GGUF metadata")


def encode_q8_0(x: np.ndarray) -> bytes:
    b = x.astype(np.float32).reshape(-1, 32)
    d = np.abs(b).max(1) / 127.0
    q = np.where(d[:, None] > 0, np.round(b / np.where(d[:, None] > 0, d[:, None], 1.0)), 0).astype(np.int8)
    out = np.empty((b.shape[0], 34), dtype=np.uint8)
    out[:, :2] = d.astype("<f2").view(np.uint8).reshape(-1, 2)
    out[:, 2:] = q.view(np.uint8)
    return out.tobytes()


def encode_q4_0(x: np.ndarray) -> bytes:
    b = x.astype(np.float32).reshape(-1, 32)
    idx = np.abs(b).argmax(1)
    mx = b[np.arange(b.shape[0]), idx]
    d = mx / -8.0
    inv = np.where(d != 0, 1.0 / np.where(d != 0, d, 1.0), 0.0)
    q = np.clip(np.round(b * inv[:, None]) + 8, 0, 15).astype(np.uint8)
    out = np.empty((b.shape[0], 18), dtype=np.uint8)
    out[:, :2] = d.astype("<f2").view(np.uint8).reshape(-1, 2)
    out[:, 2:] = q[:, :16] | (q[:, 16:] << 4)
    return out.tobytes()


def write_gguf(path, metadata: dict, tensors: dict[str, tuple[np.ndarray, int]], alignment: int = 32) -> None:
    """``tensors``: name -> (float array, ggml type among F32 / F16 / BF16 / Q8_0 / Q4_0)."""
    blobs, infos, off = [], [], 0
    for name, (arr, kind) in tensors.items():
        a = np.ascontiguousarray(arr, dtype=np.float32)
        if kind == GGML_F32:
            raw = a.astype("<f4").tobytes()
        elif kind == GGML_F16:
            raw = a.astype("<f2").tobytes()
        elif kind == GGML_BF16:
            raw = (a.view(np.uint32) >> 16).astype("<u2").tobytes()
        elif kind == GGML_Q8_0:
            raw = encode_q8_0(a)
        elif kind == GGML_Q4_0:
            raw = encode_q4_0(a)
        else:
            raise NotImplementedError(kind)
        infos.append(_pack_string(name) + struct.pack("<I", a.ndim) + b"".join(struct.pack("<Q", d) for d in reversed(a.shape)) +
                     struct.pack("<IQ", kind, off))
        pad = (-len(raw)) % alignment
        blobs.append(raw + b"\0" * pad)
        off += len(raw) + pad
    md = dict(metadata)
    md.setdefault("general.alignment", alignment)
    head = MAGIC + struct.pack("<IQQ", 3, len(tensors), len(md))
    head += b"".join(_pack_string(k) + _pack_value(v) for k, v in md.items())
    head += b"".join(infos)
    head += b"\0" * ((-len(head)) % alignment)
    Path(path).write_bytes(head + b"".join(blobs))
