"""NINT: neuron-anchored affine integer codes (1..8 bit) and their blob codec.

Math (per output row ``r``, group ``g`` of ``gs`` inputs)::

    w[r, g*gs + i] = d[r] * ls[r, g] * q[r, g, i]  -  dmin[r] * lm[r, g]

``d`` / ``dmin`` are fp16 anchors per row, ``ls`` / ``lm`` are k-bit group
codes, ``q`` are b-bit element codes.  The NINTv2 payload lets every row pick
its own ``q`` width (3-bit selector, width = selector + 1) and ``k`` width
(2-bit selector, width = nominal_k - 1 + selector).

Blob layout (little endian), matching the reference writer
(``mfq/formats/io.py:381-408``; metadata/code streams ``:200-318``)::

    u8  bits | 0x80          nominal q width, high bit marks NINTv2 storage
    u8  sub_bits             nominal k width
    i32 groupsize, i32 axis, i32 neuron_len
    u32 ndim, i64 shape[ndim], u32 out, u32 groups
    f16 d[out], f16 dmin[out]
    k-selectors (out x 2 bit), then per selector class present:
        ls stream, lm stream of the rows in that class (row order)
    q-selectors (out x 3 bit), then per selector class present:
        q stream of the rows in that class (row order)
"""

from __future__ import annotations

import struct
from dataclasses import dataclass

import numpy as np

from .bitstream import pack_bits, unpack_bits

NINT_DTYPE = "NINT"
_V2_FLAG = 0x80
_K_SEL_BITS = 2
_Q_SEL_BITS = 3
_HEAD = struct.Struct("<BBiii")

__all__ = ["NINT_DTYPE", "NintSpec", "NintTensor", "pack_nint", "unpack_nint", "dequantize_nint"]


@dataclass(frozen=True)
class NintSpec:
    """Nominal widths of one NINT tensor (default = the 4-bit gs24/k6 preset)."""

    bits: int = 4
    groupsize: int = 24
    sub_bits: int = 6

    def __post_init__(self) -> None:
        if not 1 <= self.bits <= 8 or not 1 <= self.sub_bits <= 8 or self.groupsize <= 0:
            raise ValueError(f"invalid NINT spec {self}")

    @property
    def qmax(self) -> int:
        return (1 << self.bits) - 1

    def bpw(self, neuron_len: int) -> float:
        """Nominal bits per weight: codes + two fp16 anchors + two group streams."""
        return self.bits + 32.0 / neuron_len + 2.0 * self.sub_bits / self.groupsize


@dataclass
class NintTensor:
    """Packed-domain NINT tensor.  ``q`` is ``[out, groups, gs]`` uint8."""

    spec: NintSpec
    shape: tuple[int, ...]
    axis: int
    neuron_len: int
    q: np.ndarray
    neuron_scale: np.ndarray  # [out] float32 holding fp16-representable values
    neuron_min: np.ndarray
    sub_scale: np.ndarray  # [out, groups] uint8
    sub_min: np.ndarray
    row_q_bits: np.ndarray | None = None  # [out] uint8, None = uniform nominal
    row_sub_bits: np.ndarray | None = None

    @property
    def out(self) -> int:
        return int(self.q.shape[0])

    @property
    def groups(self) -> int:
        return int(self.q.shape[1])

    def q_widths(self) -> np.ndarray:
        if self.row_q_bits is None:
            return np.full(self.out, self.spec.bits, dtype=np.uint8)
        return np.asarray(self.row_q_bits, dtype=np.uint8)

    def k_widths(self) -> np.ndarray:
        if self.row_sub_bits is None:
            return np.full(self.out, self.spec.sub_bits, dtype=np.uint8)
        return np.asarray(self.row_sub_bits, dtype=np.uint8)

    def bits_per_weight(self) -> float:
        qw = self.q_widths().astype(np.float64)
        kw = self.k_widths().astype(np.float64)
        total = (
            self.groups * self.spec.groupsize * qw.sum()
            + 2.0 * self.groups * kw.sum()
            + self.out * (32.0 + _K_SEL_BITS + _Q_SEL_BITS)
        )
        return float(total / (self.out * self.neuron_len))


def pack_nint(t: NintTensor) -> bytes:
    spec = t.spec
    out, groups, gs = t.q.shape
    if gs != spec.groupsize:
        raise ValueError("q group width does not match spec.groupsize")
    qw = t.q_widths()
    kw = t.k_widths()
    k_sel = kw.astype(np.int16) - (spec.sub_bits - 1)
    if k_sel.min(initial=0) < 0 or k_sel.max(initial=0) > 3 or qw.min(initial=1) < 1 or qw.max(initial=1) > 8:
        raise ValueError("per-row NINT widths outside the representable selector range")
    d = np.asarray(t.neuron_scale, dtype=np.float32).astype(np.float16)
    dm = np.asarray(t.neuron_min, dtype=np.float32).astype(np.float16)
    if not (np.isfinite(d).all() and np.isfinite(dm).all()):
        raise ValueError("NINT anchors must be finite in fp16")
    parts = [
        _HEAD.pack(spec.bits | _V2_FLAG, spec.sub_bits, spec.groupsize, int(t.axis), int(t.neuron_len)),
        struct.pack("<I", len(t.shape)),
        struct.pack(f"<{len(t.shape)}q", *t.shape),
        struct.pack("<II", out, groups),
        d.tobytes(),
        dm.tobytes(),
        pack_bits(k_sel.astype(np.uint8), _K_SEL_BITS),
    ]
    for sel in range(1 << _K_SEL_BITS):
        rows = np.flatnonzero(k_sel == sel)
        if rows.size:
            width = spec.sub_bits - 1 + sel
            parts.append(pack_bits(t.sub_scale[rows], width))
            parts.append(pack_bits(t.sub_min[rows], width))
    parts.append(pack_bits((qw - 1).astype(np.uint8), _Q_SEL_BITS))
    for sel in range(1 << _Q_SEL_BITS):
        rows = np.flatnonzero(qw == sel + 1)
        if rows.size:
            parts.append(pack_bits(t.q[rows], sel + 1))
    return b"".join(parts)


def unpack_nint(blob) -> NintTensor:
    raw_bits, sub_bits, gs, axis, neuron_len = _HEAD.unpack_from(blob, 0)
    if not raw_bits & _V2_FLAG:
        return _unpack_nint_v1(blob)
    bits = raw_bits & ~_V2_FLAG
    spec = NintSpec(bits=bits, groupsize=gs, sub_bits=sub_bits)
    off = _HEAD.size
    (ndim,) = struct.unpack_from("<I", blob, off)
    off += 4
    shape = tuple(struct.unpack_from(f"<{ndim}q", blob, off))
    off += 8 * ndim
    out, groups = struct.unpack_from("<II", blob, off)
    off += 8
    d = np.frombuffer(blob, dtype=np.float16, count=out, offset=off).astype(np.float32)
    off += 2 * out
    dm = np.frombuffer(blob, dtype=np.float16, count=out, offset=off).astype(np.float32)
    off += 2 * out
    if not (np.isfinite(d).all() and np.isfinite(dm).all()):
        raise ValueError("NINT anchors must be finite")
    k_sel, off = unpack_bits(blob, off, out, _K_SEL_BITS)
    kw = k_sel.astype(np.int16) + (sub_bits - 1)
    if kw.min(initial=1) < 1 or kw.max(initial=1) > 8:
        raise ValueError("invalid NINT per-row group-code width")
    ls = np.zeros((out, groups), dtype=np.uint8)
    lm = np.zeros((out, groups), dtype=np.uint8)
    for sel in range(1 << _K_SEL_BITS):
        rows = np.flatnonzero(k_sel == sel)
        if rows.size:
            width = sub_bits - 1 + sel
            a, off = unpack_bits(blob, off, rows.size * groups, width)
            b, off = unpack_bits(blob, off, rows.size * groups, width)
            ls[rows] = a.reshape(rows.size, groups)
            lm[rows] = b.reshape(rows.size, groups)
    q_sel, off = unpack_bits(blob, off, out, _Q_SEL_BITS)
    q = np.zeros((out, groups, gs), dtype=np.uint8)
    for sel in range(1 << _Q_SEL_BITS):
        rows = np.flatnonzero(q_sel == sel)
        if rows.size:
            v, off = unpack_bits(blob, off, rows.size * groups * gs, sel + 1)
            q[rows] = v.reshape(rows.size, groups, gs)
    if off != len(blob):
        raise ValueError(f"NINT blob has {len(blob) - off} trailing bytes")
    return NintTensor(
        spec=spec, shape=shape, axis=axis, neuron_len=neuron_len, q=q,
        neuron_scale=d, neuron_min=dm, sub_scale=ls, sub_min=lm,
        row_q_bits=(q_sel + 1).astype(np.uint8), row_sub_bits=kw.astype(np.uint8),
    )


def _unpack_nint_v1(blob) -> NintTensor:
    """Uniform-width predecessor layout: ls stream, lm stream, q stream."""
    bits, sub_bits, gs, axis, neuron_len = _HEAD.unpack_from(blob, 0)
    spec = NintSpec(bits=bits, groupsize=gs, sub_bits=sub_bits)
    off = _HEAD.size
    (ndim,) = struct.unpack_from("<I", blob, off)
    off += 4
    shape = tuple(struct.unpack_from(f"<{ndim}q", blob, off))
    off += 8 * ndim
    out, groups = struct.unpack_from("<II", blob, off)
    off += 8
    d = np.frombuffer(blob, dtype=np.float16, count=out, offset=off).astype(np.float32)
    off += 2 * out
    dm = np.frombuffer(blob, dtype=np.float16, count=out, offset=off).astype(np.float32)
    off += 2 * out
    ls, off = unpack_bits(blob, off, out * groups, sub_bits)
    lm, off = unpack_bits(blob, off, out * groups, sub_bits)
    q, off = unpack_bits(blob, off, out * groups * gs, bits)
    if off != len(blob):
        raise ValueError("invalid NINT v1 blob size")
    return NintTensor(
        spec=spec, shape=shape, axis=axis, neuron_len=neuron_len,
        q=q.reshape(out, groups, gs).astype(np.uint8), neuron_scale=d, neuron_min=dm,
        sub_scale=ls.reshape(out, groups).astype(np.uint8), sub_min=lm.reshape(out, groups).astype(np.uint8),
    )


def dequantize_nint_rows(t: NintTensor) -> np.ndarray:
    """Reconstruct the ``[out, neuron_len]`` float32 matrix."""
    scale = t.neuron_scale[:, None].astype(np.float32) * t.sub_scale.astype(np.float32)
    shift = t.neuron_min[:, None].astype(np.float32) * t.sub_min.astype(np.float32)
    rows = scale[:, :, None] * t.q.astype(np.float32) - shift[:, :, None]
    return rows.reshape(t.out, -1)[:, : t.neuron_len]


def dequantize_nint(t: NintTensor) -> np.ndarray:
    """Reconstruct the tensor in its logical shape (the quantized axis restored)."""
    rows = dequantize_nint_rows(t)
    shape, axis = tuple(t.shape), t.axis
    moved = (shape[axis],) + shape[:axis] + shape[axis + 1 :]
    return np.moveaxis(rows.reshape(moved), 0, axis)
