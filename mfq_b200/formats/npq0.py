"""NPQ0-S / NPQ0-L: neuron-anchored product quantization below and around one bit per weight.

A row (output neuron) is cut into 8-weight vectors, each stored as ONE index into a product of two small int8 codebooks
of 4-D halves: ``first[state][index & 7]`` and ``second[state][index >> 3]``.  Three consecutive vectors (a group of 24
weights) share a state, which selects both the codebook pair and a relative scale from a small table; one fp16 anchor
per row fixes the absolute scale:  ``w = anchor * scale_lut[state] * concat(first, second)``.

    variant   states   index bits (first + second)   code bits per weight
    NPQ0-S    4 (2 b)  3 + 3                          6/8 + 2/24 = 0.833
    NPQ0-L    8 (3 b)  3 + 4                          7/8 + 3/24 = 1.0

Blob layout (byte-compatible with ``mfq/formats/npq0_s.py:265-330`` and ``npq0_l.py:285-405`` of the reference)::

    magic "NPQS"/"NPQL"  u8 version (2 / 1)  u8 state_bits  u16 groupsize=24  i32 axis  i32 neuron_len  u32 ndim
    i64 shape[ndim]  u32 rows
    tables: 64-byte header {u8 table version (2 / 1), states, first bits, second bits, 24, 8, 0, 0, f16 scale_lut[states], 0...}
            int8 first[states][8][4]  int8 second[states][2**second bits][4]
    f16 anchors[rows]   states, LSB-first bit stream   indices, LSB-first bit stream

The dequantizer restates ``mfq/quantize/npq0_s.py:896-920`` / ``npq0_l.py:820-845``.  :func:`quantize_npq0` is this
repository's encoder: anchors from the row's largest group norm, states by a scale ladder, codebooks by a few rounds of
Lloyd iterations on the tensor itself (the reference trains its tables offline on whole models).
"""

from __future__ import annotations

import math
import struct
from dataclasses import dataclass

import numpy as np

from .bitstream import pack_bits, unpack_bits

GROUP, VEC, SUB = 24, 8, 4
_HEADER = struct.Struct("<4sBBHiiI")
_TABLE_HEADER = 64


@dataclass(frozen=True)
class Npq0Variant:
    label: str
    magic: bytes
    version: int
    table_version: int
    state_bits: int
    first_bits: int
    second_bits: int

    @property
    def states(self) -> int:
        return 1 << self.state_bits

    @property
    def index_bits(self) -> int:
        return self.first_bits + self.second_bits

    @property
    def table_bytes(self) -> int:
        return _TABLE_HEADER + self.states * ((1 << self.first_bits) + (1 << self.second_bits)) * SUB

    def bits_per_weight(self, rows: int, cols: int, include_tables: bool = True) -> float:
        groups, vecs = math.ceil(cols / GROUP), cols // VEC
        nbytes = 2 * rows + (rows * groups * self.state_bits + 7) // 8 + (rows * vecs * self.index_bits + 7) // 8
        return 8.0 * (nbytes + (self.table_bytes if include_tables else 0)) / (rows * cols)


NPQ0_S = Npq0Variant("NPQ0-S", b"NPQS", 2, 2, 2, 3, 3)
NPQ0_L = Npq0Variant("NPQ0-L", b"NPQL", 1, 1, 3, 3, 4)
VARIANTS = {v.label: v for v in (NPQ0_S, NPQ0_L)}
_BY_MAGIC = {v.magic: v for v in (NPQ0_S, NPQ0_L)}


@dataclass
class Npq0Tensor:
    variant: Npq0Variant
    shape: tuple[int, ...]
    axis: int
    neuron_len: int
    neuron_scale: np.ndarray  # [rows] fp32 (stored as fp16, non-negative)
    scale_lut: np.ndarray  # [states] fp32 (stored as fp16)
    state: np.ndarray  # [rows, groups] uint8
    indices: np.ndarray  # [rows, vectors] uint8
    first_codebooks: np.ndarray  # [states, 2**first_bits, 4] int8
    second_codebooks: np.ndarray  # [states, 2**second_bits, 4] int8

    @property
    def dtype(self) -> str:
        return self.variant.label


def _check(t: Npq0Tensor) -> tuple[int, int, int]:
    v = t.variant
    rows = int(np.asarray(t.neuron_scale).size)
    if t.neuron_len <= 0 or t.neuron_len % VEC or int(np.prod(t.shape)) != rows * t.neuron_len or not 0 <= t.axis < len(t.shape):
        raise ValueError(f"{v.label}: shape {t.shape} / axis {t.axis} / row length {t.neuron_len} are inconsistent")
    groups, vecs = math.ceil(t.neuron_len / GROUP), t.neuron_len // VEC
    anchors = np.asarray(t.neuron_scale, dtype=np.float32).astype(np.float16)
    if not np.isfinite(anchors).all() or np.signbit(anchors).any():
        raise ValueError(f"{v.label}: anchors must be finite and non-negative in fp16")
    if np.asarray(t.state).shape != (rows, groups) or np.asarray(t.indices).shape != (rows, vecs):
        raise ValueError(f"{v.label}: state / index arrays have the wrong shape")
    if np.any(np.asarray(t.state) >= v.states) or np.any(np.asarray(t.indices) >= (1 << v.index_bits)):
        raise ValueError(f"{v.label}: state or index out of range")
    lut = np.asarray(t.scale_lut, dtype=np.float32)
    if lut.shape != (v.states,) or not np.isfinite(lut).all() or np.any(lut < 0) or lut.max() <= 0:
        raise ValueError(f"{v.label}: the scale table must hold {v.states} finite non-negative values, not all zero")
    for cb, bits in ((t.first_codebooks, v.first_bits), (t.second_codebooks, v.second_bits)):
        a = np.asarray(cb)
        if a.shape != (v.states, 1 << bits, SUB) or not np.array_equal(a, np.rint(a)) or np.any(np.abs(a) > 127):
            raise ValueError(f"{v.label}: codebooks must be int8-valued [{v.states}, {1 << bits}, {SUB}] arrays")
    return rows, groups, vecs


def pack_tables(v: Npq0Variant, scale_lut, first, second) -> bytes:
    """One table set as it sits in a blob: the 64-byte header with the scale ladder, then both int8 codebooks."""
    head = bytearray(_TABLE_HEADER)
    head[0:6] = bytes([v.table_version, v.states, v.first_bits, v.second_bits, GROUP, VEC])
    head[8 : 8 + 2 * v.states] = np.asarray(scale_lut, dtype=np.float32).astype("<f2").tobytes()
    return bytes(head) + np.asarray(first, dtype=np.int8).tobytes() + np.asarray(second, dtype=np.int8).tobytes()


def unpack_tables(v: Npq0Variant, raw) -> tuple[np.ndarray, np.ndarray, np.ndarray]:
    """Inverse of :func:`pack_tables` over exactly ``v.table_bytes`` bytes: (scale ladder fp32, first, second)."""
    raw = bytes(raw)
    if len(raw) != v.table_bytes:
        raise ValueError(f"{v.label}: a table set is {v.table_bytes} bytes, got {len(raw)}")
    head = raw[:_TABLE_HEADER]
    if tuple(head[:6]) != (v.table_version, v.states, v.first_bits, v.second_bits, GROUP, VEC) or any(head[6:8]) or \
            any(head[8 + 2 * v.states :]):
        raise ValueError(f"{v.label}: unsupported table profile")
    lut = np.frombuffer(head, dtype="<f2", count=v.states, offset=8).astype(np.float32)
    n1 = v.states * (1 << v.first_bits) * SUB
    first = np.frombuffer(raw, dtype=np.int8, count=n1, offset=_TABLE_HEADER).reshape(v.states, 1 << v.first_bits, SUB).copy()
    second = np.frombuffer(raw, dtype=np.int8, offset=_TABLE_HEADER + n1).reshape(v.states, 1 << v.second_bits, SUB).copy()
    return lut, first, second


def _pack_tables(t: Npq0Tensor) -> bytes:
    return pack_tables(t.variant, t.scale_lut, t.first_codebooks, t.second_codebooks)


def pack_npq0(t: Npq0Tensor) -> bytes:
    rows, _g, _v = _check(t)
    v = t.variant
    shape = tuple(int(s) for s in t.shape)
    return b"".join([
        _HEADER.pack(v.magic, v.version, v.state_bits, GROUP, t.axis, t.neuron_len, len(shape)),
        struct.pack(f"<{len(shape)}q", *shape), struct.pack("<I", rows), _pack_tables(t),
        np.asarray(t.neuron_scale, dtype=np.float32).astype("<f2").tobytes(),
        pack_bits(np.asarray(t.state, dtype=np.uint8).reshape(-1), v.state_bits),
        pack_bits(np.asarray(t.indices, dtype=np.uint8).reshape(-1), v.index_bits)])


def unpack_npq0(blob) -> Npq0Tensor:
    blob = memoryview(blob)
    if len(blob) < _HEADER.size:
        raise ValueError("truncated NPQ0 header")
    magic, version, state_bits, groupsize, axis, neuron_len, ndim = _HEADER.unpack_from(blob)
    v = _BY_MAGIC.get(bytes(magic))
    if v is None or version != v.version or state_bits != v.state_bits or groupsize != GROUP:
        raise ValueError("not an NPQ0-S / NPQ0-L blob of a known version")
    if ndim <= 0 or neuron_len <= 0 or neuron_len % VEC:
        raise ValueError(f"{v.label}: invalid dimensions")
    off = _HEADER.size
    shape = tuple(struct.unpack_from(f"<{ndim}q", blob, off))
    off += 8 * ndim
    rows = struct.unpack_from("<I", blob, off)[0]
    off += 4
    if off + v.table_bytes > len(blob):
        raise ValueError(f"{v.label}: truncated tables")
    lut, first, second = unpack_tables(v, blob[off : off + v.table_bytes])
    off += v.table_bytes
    anchors = np.frombuffer(blob, dtype="<f2", count=rows, offset=off).astype(np.float32)
    off += 2 * rows
    groups, vecs = math.ceil(neuron_len / GROUP), neuron_len // VEC
    state, off = unpack_bits(blob, off, rows * groups, v.state_bits)
    idx, off = unpack_bits(blob, off, rows * vecs, v.index_bits)
    if off != len(blob):
        raise ValueError(f"{v.label}: {len(blob) - off} stray bytes after the index stream")
    t = Npq0Tensor(v, shape, axis, neuron_len, anchors, lut, state.reshape(rows, groups), idx.reshape(rows, vecs), first, second)
    _check(t)
    return t


def dequantize_npq0(t: Npq0Tensor) -> np.ndarray:
    rows, groups, vecs = _check(t)
    v = t.variant
    idx = np.zeros((rows, groups * 3), dtype=np.uint8)
    idx[:, :vecs] = t.indices
    vstate = np.repeat(np.asarray(t.state, dtype=np.uint8), 3, axis=1)
    first = np.asarray(t.first_codebooks, dtype=np.int8)[vstate, idx & ((1 << v.first_bits) - 1)]
    second = np.asarray(t.second_codebooks, dtype=np.int8)[vstate, idx >> v.first_bits]
    code = np.concatenate([first, second], -1).reshape(rows, -1)[:, : t.neuron_len]
    scale = np.asarray(t.neuron_scale, dtype=np.float32)[:, None] * np.asarray(t.scale_lut, dtype=np.float32)[np.asarray(t.state)]
    m = code.astype(np.float32) * np.repeat(scale, GROUP, axis=1)[:, : t.neuron_len]
    moved = (t.shape[t.axis],) + tuple(s for i, s in enumerate(t.shape) if i != t.axis)
    return np.moveaxis(m.reshape(moved), 0, t.axis)


def quantize_npq0(weight, variant: Npq0Variant | str = NPQ0_L, *, axis: int = 0, iterations: int = 6, seed: int = 0) -> Npq0Tensor:
    """Encode ``weight`` (rank >= 2, ``axis`` = output neurons, row length a multiple of 8).  Anchor = the row's largest
    group RMS mapped to the top of the scale ladder; a group's state = the ladder step nearest its RMS; the codebook pair
    of every state is fitted by Lloyd iterations over that state's (scale-normalised) half-vectors."""
    v = VARIANTS[variant] if isinstance(variant, str) else variant
    w = np.asarray(weight, dtype=np.float32)
    axis %= w.ndim
    rows_m = np.moveaxis(w, axis, 0).reshape(w.shape[axis], -1)
    rows, n = rows_m.shape
    if n % VEC:
        raise ValueError(f"{v.label}: the row length must be a multiple of 8")
    groups, vecs = math.ceil(n / GROUP), n // VEC
    pad = np.zeros((rows, groups * GROUP), dtype=np.float32)
    pad[:, :n] = rows_m
    g = pad.reshape(rows, groups, GROUP)
    valid = np.minimum(GROUP, n - GROUP * np.arange(groups)).astype(np.float32)
    rms = np.sqrt((g ** 2).sum(-1) / valid[None, :])
    ladder = 2.0 ** (-np.arange(v.states - 1, -1, -1, dtype=np.float32) * (4.0 / max(1, v.states - 1)))  # top step = 1
    lut = ladder.astype(np.float16).astype(np.float32)
    top = rms.max(1)
    anchors = (top / 48.0).astype(np.float16).astype(np.float32)  # a unit-RMS group at full scale uses codes of magnitude ~48
    anchors[anchors == 0] = np.float32(np.float16(6e-5))
    ratio = rms / np.maximum(top[:, None], 1e-30)
    state = np.abs(np.log2(np.maximum(ratio[..., None], 1e-12)) - np.log2(lut)[None, None, :]).argmin(-1).astype(np.uint8)
    scale = anchors[:, None] * lut[state]
    norm = (g / np.maximum(scale[..., None], 1e-30)).reshape(rows, groups * 3, 2, SUB)  # halves in code units
    vstate = np.repeat(state, 3, axis=1)
    live = (np.arange(groups * 3) < vecs)[None, :].repeat(rows, 0)
    rng = np.random.default_rng(seed)
    books = []
    idx_parts = []
    for half, bits in ((0, v.first_bits), (1, v.second_bits)):
        k = 1 << bits
        cb = np.zeros((v.states, k, SUB), dtype=np.float32)
        assign = np.zeros((rows, groups * 3), dtype=np.uint8)
        for s in range(v.states):
            sel = (vstate == s) & live
            pts = norm[:, :, half][sel]
            if pts.shape[0] == 0:
                continue
            cent = pts[rng.choice(pts.shape[0], size=k, replace=pts.shape[0] < k)].copy()
            for _ in range(iterations):
                d = ((pts[:, None, :] - cent[None]) ** 2).sum(-1)
                a = d.argmin(1)
                for j in range(k):
                    m = a == j
                    if m.any():
                        cent[j] = pts[m].mean(0)
            cent = np.clip(np.rint(cent), -127, 127)
            d = ((pts[:, None, :] - cent[None]) ** 2).sum(-1)
            assign[sel] = d.argmin(1).astype(np.uint8)
            cb[s] = cent
        books.append(cb.astype(np.int8))
        idx_parts.append(assign)
    indices = (idx_parts[0] | (idx_parts[1] << v.first_bits))[:, :vecs].astype(np.uint8)
    return Npq0Tensor(v, tuple(w.shape), axis, n, anchors, lut, state, indices, books[0], books[1])
