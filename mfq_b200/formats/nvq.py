"""NVQ: neuron-anchored lattice vector codes and their blob codec.

Math (row ``r``, group ``g`` of ``gs`` inputs, vector ``v`` of 8 (E8) or 4 (D4)
inputs)::

    w[r, i] = d[r] * s[r, i // gs] * C[index[r, i // vec]][i % vec] * sign[r, i]

``C`` holds odd positive integer magnitudes.  Signs are stored as 7 bits per 8
weights; the 8th sign is the parity of the stored 7 ("even" mode) or that parity
XOR bit 7 of the vector index ("index_parity" mode, E8-256 only).

The three base magnitude grids are the public ``kgrid_2bit_256`` / ``kgrid_256``
/ ``kgrid_512`` tables of llama.cpp's IQ2/IQ3 quantizers (MIT licence); they are
shipped as a data file because the container stores only indices into them.  The
larger grids are derived deterministically from them (see
:func:`_grow_codebook`).  Layout parity: ``mfq/formats/nvq.py:791-858`` (plain)
and ``:425-520,659-757,861-930`` (JSC) in the reference.

Plain blob::

    "NVQ1" u8 id|flags  u8 sub_bits  u16 groupsize  i32 axis  i32 neuron_len  u32 ndim
    i64 shape[ndim]  u32 out  [custom codebook: entries x u16]  f16 d[out]
    s stream (out*ceil(K/gs) x sub_bits)  index stream (out*ceil(K/vec) x index_bits)
    sign stream (out*ceil(K/8) x 7)

JSC blob (flag 0x20, gs 24, 4-bit state per group): 64-byte metadata
``[version, banks, 16, analytic, scale_lut 16xf16, bank_for_state 16xu8, group64 flag, pad]``,
``banks*entries*vec`` int8 codebook banks, anchors, then either the three streams
(state, index, sign) or one u64 record per 24-weight group ("group64")::

    w = d[r] * scale_lut[state] * banks[bank_for_state[state]][index] * sign
"""

from __future__ import annotations

import hashlib
import math
import struct
from dataclasses import dataclass
from pathlib import Path

import numpy as np

from .bitstream import pack_bits, unpack_bits

NVQ_DTYPE = "NVQ"
_MAGIC = b"NVQ1"
_OLD_MAGIC = b"NIQ1"
_HEAD = struct.Struct("<4sBBHiiI")
_FLAG_INDEX_PARITY = 0x80
_FLAG_CUSTOM = 0x40
_FLAG_JSC = 0x20
_IDS = {"e8_256": 1, "d4_256": 2, "d4_512": 3, "e8_1024": 4, "e8_4096": 5, "d4_1024": 6}
_NAMES = {v: k for k, v in _IDS.items()}
_INDEX_BITS = {"e8_256": 8, "e8_1024": 10, "e8_4096": 12, "d4_256": 8, "d4_512": 9, "d4_1024": 10}
_GRID_SHA256 = "0c0f6347fde493d8ac0bdb6067175d2d2276948ecb8731bc377ae2383fc792d6"

__all__ = [
    "NVQ_DTYPE", "NvqSpec", "NvqTensor", "NvqJscTensor", "codebook", "pack_nvq", "unpack_nvq",
    "dequantize_nvq", "decode_signs",
]


def _load_base_grids() -> dict[str, np.ndarray]:
    raw = (Path(__file__).parent / "data" / "lattice_grids.bin").read_bytes()
    if hashlib.sha256(raw).hexdigest() != _GRID_SHA256:
        raise RuntimeError("lattice grid data file is corrupt")
    a = np.frombuffer(raw, dtype=np.int8)
    return {
        "e8_256": a[:2048].reshape(256, 8).copy(),
        "d4_256": a[2048:3072].reshape(256, 4).copy(),
        "d4_512": a[3072:].reshape(512, 4).copy(),
    }


def _reverse_bits(x: np.ndarray, width: int) -> np.ndarray:
    y = np.zeros_like(x)
    for b in range(width):
        y |= ((x >> b) & 1) << (width - 1 - b)
    return y


def _grow_codebook(base: np.ndarray, entries: int) -> np.ndarray:
    """Append unused lattice points in bit-reversed id order until ``entries`` rows.

    A point with digits ``t_j = (c_j - 1) / 2`` has id ``sum t_j << (j*digit_bits)``
    (2 digit bits for 8-D, 3 for 4-D).  Walking ids in bit-reversed order spreads
    the additions over the whole lattice cube; existing rows keep their index.
    """
    dims = base.shape[1]
    digit_bits = 2 if dims == 8 else 3
    width = dims * digit_bits
    shifts = (digit_bits * np.arange(dims)).astype(np.uint32)
    have = ((base.astype(np.uint32) - 1) // 2) << shifts[None, :]
    have_ids = np.bitwise_or.reduce(have, axis=1)
    taken = np.zeros(1 << width, dtype=bool)
    taken[have_ids] = True
    walk = _reverse_bits(np.arange(1 << width, dtype=np.uint32), width)
    extra = walk[~taken[walk]][: entries - base.shape[0]]
    ids = np.concatenate([have_ids, extra])
    digits = (ids[:, None] >> shifts[None, :]) & ((1 << digit_bits) - 1)
    return np.ascontiguousarray(2 * digits + 1, dtype=np.int8)


_GRIDS = _load_base_grids()
_GRIDS["e8_1024"] = _grow_codebook(_GRIDS["e8_256"], 1024)
_GRIDS["e8_4096"] = _grow_codebook(_GRIDS["e8_1024"], 4096)
_GRIDS["d4_1024"] = _grow_codebook(_GRIDS["d4_512"], 1024)


@dataclass(frozen=True)
class NvqSpec:
    codebook: str
    groupsize: int = 24
    sub_bits: int = 4
    sign_mode: str = "even"

    def __post_init__(self) -> None:
        if self.codebook not in _IDS:
            raise ValueError(f"unknown NVQ codebook {self.codebook!r}")
        if self.groupsize <= 0 or self.groupsize % 8:
            raise ValueError("NVQ groupsize must be a positive multiple of 8")
        if not 1 <= self.sub_bits <= 8:
            raise ValueError("NVQ sub_bits must be in 1..8")
        if self.sign_mode not in ("even", "index_parity"):
            raise ValueError(f"unknown NVQ sign mode {self.sign_mode!r}")
        if self.sign_mode == "index_parity" and self.codebook != "e8_256":
            raise ValueError("index_parity signs need the 256-entry E8 grid")

    @property
    def vector_size(self) -> int:
        return 8 if self.codebook.startswith("e8") else 4

    @property
    def index_bits(self) -> int:
        return _INDEX_BITS[self.codebook]

    @property
    def entries(self) -> int:
        return 1 << self.index_bits

    def payload_nbytes(self, out: int, neuron_len: int) -> int:
        ng = math.ceil(neuron_len / self.groupsize)
        nvec = math.ceil(neuron_len / self.vector_size)
        nsign = math.ceil(neuron_len / 8)
        return (
            2 * out + (out * ng * self.sub_bits + 7) // 8
            + (out * nvec * self.index_bits + 7) // 8 + (out * nsign * 7 + 7) // 8
        )

    def bpw(self, neuron_len: int, out: int = 1) -> float:
        return 8.0 * self.payload_nbytes(out, neuron_len) / (out * neuron_len)


NVQ2_E8 = NvqSpec("e8_256")
NVQ3_D4 = NvqSpec("d4_256")
NVQ3_D4_512 = NvqSpec("d4_512")
NVQ3_D4_1024 = NvqSpec("d4_1024")


def codebook(spec_or_name) -> np.ndarray:
    name = spec_or_name.codebook if isinstance(spec_or_name, NvqSpec) else spec_or_name
    return _GRIDS[name]


def _check_codebook(spec: NvqSpec, table: np.ndarray) -> np.ndarray:
    t = np.asarray(table)
    if t.shape != (spec.entries, spec.vector_size):
        raise ValueError(f"NVQ codebook shape {t.shape} != {(spec.entries, spec.vector_size)}")
    top = 7 if spec.vector_size == 8 else 15
    ti = np.rint(t).astype(np.int16)
    if not np.array_equal(ti, t) or ti.min() < 1 or ti.max() > top or np.any((ti & 1) == 0):
        raise ValueError(f"NVQ codebook entries must be odd integers in [1, {top}]")
    return ti.astype(np.int8)


def _codebook_to_bytes(spec: NvqSpec, table: np.ndarray) -> bytes:
    t = _check_codebook(spec, table)
    digit_bits = 2 if spec.vector_size == 8 else 3
    shifts = (digit_bits * np.arange(spec.vector_size)).astype(np.uint16)
    digits = ((t.astype(np.uint16) - 1) // 2) << shifts[None, :]
    return np.bitwise_or.reduce(digits, axis=1).astype("<u2").tobytes()


def _codebook_from_bytes(spec: NvqSpec, payload) -> np.ndarray:
    ids = np.frombuffer(payload, dtype="<u2", count=spec.entries)
    digit_bits = 2 if spec.vector_size == 8 else 3
    shifts = (digit_bits * np.arange(spec.vector_size)).astype(np.uint16)
    digits = (ids[:, None] >> shifts[None, :]) & ((1 << digit_bits) - 1)
    return _check_codebook(spec, 2 * digits + 1)


@dataclass
class NvqTensor:
    spec: NvqSpec
    shape: tuple[int, ...]
    axis: int
    neuron_len: int
    neuron_scale: np.ndarray  # [out] float32 (fp16-representable, >= 0)
    sub_scale: np.ndarray  # [out, ceil(K/gs)] uint8
    indices: np.ndarray  # [out, ceil(K/vec)] uint8/uint16
    signs: np.ndarray  # [out, ceil(K/8)] uint8 (7 significant bits)
    codebook: np.ndarray | None = None

    @property
    def out(self) -> int:
        return int(np.asarray(self.neuron_scale).size)


@dataclass
class NvqJscTensor:
    """NVQ with a joint scale/codebook state per 24-weight group."""

    base_spec: NvqSpec
    shape: tuple[int, ...]
    axis: int
    neuron_len: int
    neuron_scale: np.ndarray
    scale_lut: np.ndarray  # [16] float32 (fp16-representable)
    bank_for_state: np.ndarray  # [16] uint8
    codebooks: np.ndarray  # [banks, entries, vec] int8
    state: np.ndarray  # [out, groups] uint8 (4 bit)
    indices: np.ndarray
    signs: np.ndarray
    storage_layout: str = "streams"  # or "group64"
    analytic: bool = False

    @property
    def out(self) -> int:
        return int(np.asarray(self.neuron_scale).size)


def _anchors_f16(x: np.ndarray) -> np.ndarray:
    a = np.asarray(x, dtype=np.float32).astype(np.float16)
    if not np.isfinite(a).all() or np.signbit(a).any():
        raise ValueError("NVQ anchors must be finite and non-negative in fp16")
    return a


def _shapes(spec: NvqSpec, neuron_len: int) -> tuple[int, int, int]:
    return (
        math.ceil(neuron_len / spec.groupsize),
        math.ceil(neuron_len / spec.vector_size),
        math.ceil(neuron_len / 8),
    )


def pack_nvq(t) -> bytes:
    if isinstance(t, NvqJscTensor):
        return _pack_jsc(t)
    spec = t.spec
    out = t.out
    ng, nvec, nsign = _shapes(spec, t.neuron_len)
    if t.sub_scale.shape != (out, ng) or t.indices.shape != (out, nvec) or t.signs.shape != (out, nsign):
        raise ValueError("NVQ stream shapes do not match neuron_len/groupsize")
    flags = _IDS[spec.codebook]
    if spec.sign_mode == "index_parity":
        flags |= _FLAG_INDEX_PARITY
    custom = b""
    if t.codebook is not None:
        flags |= _FLAG_CUSTOM
        custom = _codebook_to_bytes(spec, t.codebook)
    return b"".join([
        _HEAD.pack(_MAGIC, flags, spec.sub_bits, spec.groupsize, int(t.axis), int(t.neuron_len), len(t.shape)),
        struct.pack(f"<{len(t.shape)}q", *t.shape),
        struct.pack("<I", out),
        custom,
        _anchors_f16(t.neuron_scale).tobytes(),
        pack_bits(t.sub_scale, spec.sub_bits),
        pack_bits(t.indices, spec.index_bits),
        pack_bits(t.signs, 7),
    ])


_JSC_META = 64


def analytic_jsc_tables(banks: int, vector_size: int) -> tuple[np.ndarray, np.ndarray]:
    """Closed-form state tables: state -> (relative scale, bank = state % banks)."""
    state = np.arange(16)
    rank = (state // banks).astype(np.float32)
    if banks == 1:
        scale = state.astype(np.float32)
    elif vector_size == 4:
        scale = rank + 1.0
    else:
        scale = 15.0 * (rank + 1.0) / (16 // banks)
    return scale.astype(np.float32), (state % banks).astype(np.uint8)


def _pack_jsc(t: NvqJscTensor) -> bytes:
    spec = t.base_spec
    if spec.groupsize != 24 or spec.sub_bits != 4 or spec.sign_mode != "even":
        raise ValueError("NVQ-JSC needs gs 24, 4-bit states and even-parity signs")
    out = t.out
    ng, nvec, nsign = _shapes(spec, t.neuron_len)
    banks = int(t.codebooks.shape[0])
    if banks not in (1, 2, 4) or t.codebooks.shape[1:] != (spec.entries, spec.vector_size):
        raise ValueError("invalid NVQ-JSC codebook banks")
    group64 = t.storage_layout == "group64"
    if group64 and spec.codebook != "e8_4096":
        raise ValueError("group64 records need the 4096-entry E8 grid")
    meta = bytearray(_JSC_META)
    lut = np.asarray(t.scale_lut, dtype=np.float32).reshape(-1)
    bank_map = np.asarray(t.bank_for_state, dtype=np.uint8).reshape(-1)
    if lut.shape != (16,) or bank_map.shape != (16,) or bank_map.max() >= banks or lut.min() < 0:
        raise ValueError("invalid NVQ-JSC state tables")
    a_lut, a_bank = analytic_jsc_tables(banks, spec.vector_size)
    analytic = np.array_equal(lut, a_lut) and np.array_equal(bank_map, a_bank)
    # byte 0 doubles as the layout version: 1 = three streams, 2 = 64-bit group records
    meta[0], meta[1], meta[2], meta[3] = (2 if group64 else 1), banks, 16, int(analytic)
    meta[4:36] = lut.astype("<f2").tobytes()
    meta[36:52] = bank_map.tobytes()
    meta[52] = 1 if group64 else 0
    head = _HEAD.pack(_MAGIC, _IDS[spec.codebook] | _FLAG_JSC, 4, 24, int(t.axis), int(t.neuron_len), len(t.shape))
    parts = [
        head, struct.pack(f"<{len(t.shape)}q", *t.shape), struct.pack("<I", out), bytes(meta),
        np.ascontiguousarray(t.codebooks, dtype=np.int8).tobytes(), _anchors_f16(t.neuron_scale).tobytes(),
    ]
    if group64:
        parts.append(_group64_records(t, out, ng).tobytes())
    else:
        parts += [pack_bits(t.state, 4), pack_bits(t.indices, spec.index_bits), pack_bits(t.signs, 7)]
    return b"".join(parts)


def _group64_records(t: NvqJscTensor, out: int, ng: int) -> np.ndarray:
    """One u64 per group: three 20-bit segments (12-bit index | 7 signs | parity) + state<<60."""
    idx = np.zeros((out, ng * 3), dtype=np.uint64)
    sgn = np.zeros((out, ng * 3), dtype=np.uint64)
    idx[:, : t.indices.shape[1]] = t.indices
    sgn[:, : t.signs.shape[1]] = t.signs
    parity = np.zeros_like(sgn)
    for b in range(7):
        parity ^= (sgn >> np.uint64(b)) & np.uint64(1)
    seg = idx | (sgn << np.uint64(12)) | (parity << np.uint64(19))
    seg = seg.reshape(out, ng, 3)
    rec = seg[:, :, 0] | (seg[:, :, 1] << np.uint64(20)) | (seg[:, :, 2] << np.uint64(40))
    rec |= np.asarray(t.state, dtype=np.uint64) << np.uint64(60)
    return rec.astype("<u8")


def unpack_nvq(blob):
    magic, flags, sub_bits, gs, axis, neuron_len, ndim = _HEAD.unpack_from(blob, 0)
    if magic not in (_MAGIC, _OLD_MAGIC):
        raise ValueError(f"bad NVQ magic {magic!r}")
    cid = flags & ~(_FLAG_INDEX_PARITY | _FLAG_CUSTOM | _FLAG_JSC)
    if cid not in _NAMES:
        raise ValueError(f"unknown NVQ codebook id {cid}")
    mode = "index_parity" if flags & _FLAG_INDEX_PARITY else "even"
    spec = NvqSpec(_NAMES[cid], groupsize=gs, sub_bits=sub_bits, sign_mode=mode)
    off = _HEAD.size
    shape = tuple(struct.unpack_from(f"<{ndim}q", blob, off))
    off += 8 * ndim
    (out,) = struct.unpack_from("<I", blob, off)
    off += 4
    ng, nvec, nsign = _shapes(spec, neuron_len)
    if flags & _FLAG_JSC:
        if flags & _FLAG_CUSTOM or mode != "even" or gs != 24 or sub_bits != 4:
            raise ValueError("invalid NVQ-JSC profile flags")
        meta = bytes(blob[off : off + _JSC_META])
        if len(meta) < _JSC_META or meta[0] not in (1, 2) or meta[1] not in (1, 2, 4) or meta[2] != 16:
            raise ValueError("invalid NVQ-JSC metadata")
        if (meta[0] == 2 and (meta[52] != 1 or any(meta[53:]))) or (meta[0] == 1 and any(meta[52:])):
            raise ValueError("invalid NVQ-JSC storage layout bytes")
        banks = meta[1]
        lut = np.frombuffer(meta, dtype="<f2", count=16, offset=4).astype(np.float32)
        bank_for_state = np.frombuffer(meta, dtype=np.uint8, count=16, offset=36).copy()
        if bank_for_state.max() >= banks:
            raise ValueError("NVQ-JSC state refers to a missing bank")
        group64 = meta[0] == 2
        off += _JSC_META
        n = banks * spec.entries * spec.vector_size
        books = np.frombuffer(blob, dtype=np.int8, count=n, offset=off).reshape(banks, spec.entries, spec.vector_size).copy()
        off += n
        d = np.frombuffer(blob, dtype=np.float16, count=out, offset=off).astype(np.float32)
        off += 2 * out
        if group64:
            rec = np.frombuffer(blob, dtype="<u8", count=out * ng, offset=off).reshape(out, ng)
            off += 8 * out * ng
            state = (rec >> np.uint64(60)).astype(np.uint8)
            segs = np.stack([(rec >> np.uint64(20 * j)) & np.uint64(0xFFFFF) for j in range(3)], axis=-1).reshape(out, ng * 3)
            indices = (segs & np.uint64(0xFFF)).astype(np.uint16)[:, :nvec]
            signs = ((segs >> np.uint64(12)) & np.uint64(0x7F)).astype(np.uint8)[:, :nsign]
        else:
            state, off = unpack_bits(blob, off, out * ng, 4)
            indices, off = unpack_bits(blob, off, out * nvec, spec.index_bits)
            signs, off = unpack_bits(blob, off, out * nsign, 7)
            state, indices, signs = state.reshape(out, ng), indices.reshape(out, nvec), signs.reshape(out, nsign)
        if off != len(blob):
            raise ValueError("invalid NVQ-JSC blob size")
        return NvqJscTensor(
            base_spec=spec, shape=shape, axis=axis, neuron_len=neuron_len, neuron_scale=d, scale_lut=lut,
            bank_for_state=bank_for_state, codebooks=books, state=state, indices=indices, signs=signs,
            storage_layout="group64" if group64 else "streams", analytic=bool(meta[3]),
        )
    table = None
    if flags & _FLAG_CUSTOM:
        table = _codebook_from_bytes(spec, blob[off : off + 2 * spec.entries])
        off += 2 * spec.entries
    d = np.frombuffer(blob, dtype=np.float16, count=out, offset=off).astype(np.float32)
    if np.signbit(d).any() or not np.isfinite(d).all():
        raise ValueError("NVQ anchors must be finite and non-negative")
    off += 2 * out
    s, off = unpack_bits(blob, off, out * ng, sub_bits)
    idx, off = unpack_bits(blob, off, out * nvec, spec.index_bits)
    sg, off = unpack_bits(blob, off, out * nsign, 7)
    if off != len(blob):
        raise ValueError(f"invalid NVQ blob size: consumed {off} of {len(blob)}")
    return NvqTensor(
        spec=spec, shape=shape, axis=axis, neuron_len=neuron_len, neuron_scale=d,
        sub_scale=s.reshape(out, ng), indices=idx.reshape(out, nvec), signs=sg.reshape(out, nsign), codebook=table,
    )


def decode_signs(signs: np.ndarray, neuron_len: int, spec: NvqSpec, indices: np.ndarray | None = None) -> np.ndarray:
    """Expand 7-bit masks to +-1 per weight (``[out, neuron_len]`` float32)."""
    m = np.asarray(signs, dtype=np.uint8)
    low = (m[..., None] >> np.arange(7, dtype=np.uint8)) & 1
    last = low.sum(axis=-1, keepdims=True).astype(np.uint8) & 1
    if spec.sign_mode == "index_parity":
        last = last ^ ((np.asarray(indices, dtype=np.uint8) >> 7) & 1)[..., None]
    neg = np.concatenate([low, last], axis=-1).reshape(m.shape[0], -1)[:, :neuron_len]
    return np.where(neg != 0, np.float32(-1.0), np.float32(1.0))


def dequantize_nvq_rows(t) -> np.ndarray:
    if isinstance(t, NvqJscTensor):
        spec = t.base_spec
        out = t.out
        vpg = spec.groupsize // spec.vector_size
        bank = t.bank_for_state[t.state]  # [out, ng]
        bank_v = np.repeat(bank, vpg, axis=1)[:, : t.indices.shape[1]]
        mag = t.codebooks[bank_v, t.indices].reshape(out, -1)[:, : t.neuron_len].astype(np.float32)
        gscale = t.neuron_scale[:, None] * t.scale_lut[t.state]
        scale = np.repeat(gscale, spec.groupsize, axis=1)[:, : t.neuron_len]
        return mag * decode_signs(t.signs, t.neuron_len, spec) * scale
    spec = t.spec
    table = _GRIDS[spec.codebook] if t.codebook is None else t.codebook
    mag = table[t.indices].reshape(t.out, -1)[:, : t.neuron_len].astype(np.float32)
    gscale = t.neuron_scale[:, None].astype(np.float32) * t.sub_scale.astype(np.float32)
    scale = np.repeat(gscale, spec.groupsize, axis=1)[:, : t.neuron_len]
    return mag * decode_signs(t.signs, t.neuron_len, spec, t.indices) * scale


def dequantize_nvq(t) -> np.ndarray:
    rows = dequantize_nvq_rows(t)
    shape, axis = tuple(t.shape), t.axis
    moved = (shape[axis],) + shape[:axis] + shape[axis + 1 :]
    return np.moveaxis(rows.reshape(moved), 0, axis)
