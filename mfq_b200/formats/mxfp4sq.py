"""MXFP4-SQ: per-row re-quantization of native MXFP4 matrices (magic ``SQV2``).

Every row carries a 2-bit ``q-1`` descriptor.  ``q = 4`` rows are the lossless
endpoint: their symbols are the native E2M1 nibbles and they keep one E8M0 scale
per 32 columns.  ``q < 4`` rows hold ``q``-bit symbols plus, per row, a binary
per-block state selector, eight 2-bit state scales and eight 5-bit palette ids.

Layout (parity: ``mfq/formats/mxfp4_sq.py:161-197,275-360`` of the reference)::

    "SQV2" u8 version=2  u8 matrix_scale_base  u16 0  u64 rows  u64 cols
    q descriptors  rows x 2 bit, zero padded to 4 bytes
    symbols        row r: cols * q_r / 8 bytes
    block selectors (sq_rows*cols/32 x 1 bit), state scales (sq_rows*8 x 2 bit),
    state palettes (sq_rows*8 x 5 bit), native E8M0 scales (sq4_rows x cols/32)

This module reads and writes the container and decodes the ``q = 4`` rows (what the
tensor-core MXFP4 path consumes).  Rows with ``q < 4`` are carried through
byte-exactly; expanding them needs the palette catalogue of the offline
re-quantizer, which is outside the serving path.
"""

from __future__ import annotations

import struct
from dataclasses import dataclass

import numpy as np

from .bitstream import pack_bits, unpack_bits, packed_nbytes
from .mx import E2M1_VALUES, MXFP4_DTYPE, MxTensor, e8m0_to_float

MXFP4_SQ_DTYPE = "MXFP4-SQ"
_HEAD = struct.Struct("<4sBBHQQ")
_MAGIC = b"SQV2"


@dataclass
class Mxfp4SqTensor:
    shape: tuple[int, int]
    matrix_scale_base: int
    row_q_bits: np.ndarray  # [rows] in 1..4
    row_symbols: list[bytes]  # per row, cols*q/8 bytes
    block_selectors: np.ndarray  # [sq_rows, cols/32] {0,1}
    state_scales: np.ndarray  # [sq_rows, 8] 0..3
    state_palettes: np.ndarray  # [sq_rows, 8] 0..31
    native_scales: np.ndarray  # [sq4_rows, cols/32] E8M0

    @property
    def is_native(self) -> bool:
        return bool(np.all(np.asarray(self.row_q_bits) == 4))


def from_mxfp4(t: MxTensor, matrix_scale_base: int = 127) -> Mxfp4SqTensor:
    """Wrap a native MXFP4 matrix as the all-SQ4 (lossless) profile."""
    if t.dtype != MXFP4_DTYPE:
        raise ValueError("expected an MXFP4 tensor")
    rows, cols = t.shape
    blocks = cols // 32
    return Mxfp4SqTensor(
        (rows, cols), matrix_scale_base, np.full(rows, 4, dtype=np.uint8),
        [np.ascontiguousarray(t.values[r]).tobytes() for r in range(rows)],
        np.empty((0, blocks), np.uint8), np.empty((0, 8), np.uint8), np.empty((0, 8), np.uint8),
        np.ascontiguousarray(t.scales, dtype=np.uint8),
    )


def pack_mxfp4sq(t: Mxfp4SqTensor) -> bytes:
    rows, cols = t.shape
    if cols % 32 or rows <= 0:
        raise ValueError("MXFP4-SQ needs a non-empty matrix of complete 32-blocks")
    q = np.asarray(t.row_q_bits, dtype=np.uint8)
    if q.shape != (rows,) or q.min() < 1 or q.max() > 4:
        raise ValueError("MXFP4-SQ q descriptors must be in 1..4, one per row")
    for r in range(rows):
        if len(t.row_symbols[r]) != cols * int(q[r]) // 8:
            raise ValueError(f"row {r} symbol stream has the wrong size")
    sel = pack_bits(q - 1, 2)
    sel += b"\0" * (((len(sel) + 3) & ~3) - len(sel))
    if np.any(np.asarray(t.native_scales) > 254):
        raise ValueError("MXFP4-SQ native scales must be valid E8M0")
    return b"".join([
        _HEAD.pack(_MAGIC, 2, int(t.matrix_scale_base), 0, rows, cols), sel, b"".join(t.row_symbols),
        pack_bits(t.block_selectors, 1) if t.block_selectors.size else b"",
        pack_bits(t.state_scales, 2) if t.state_scales.size else b"",
        pack_bits(t.state_palettes, 5) if t.state_palettes.size else b"",
        np.ascontiguousarray(t.native_scales, dtype=np.uint8).tobytes(),
    ])


def unpack_mxfp4sq(blob) -> Mxfp4SqTensor:
    magic, version, base, reserved, rows, cols = _HEAD.unpack_from(blob, 0)
    if magic != _MAGIC or version != 2 or reserved or cols % 32 or rows <= 0:
        raise ValueError("unsupported MXFP4-SQ payload (only the adaptive SQV2 layout is read)")
    off = _HEAD.size
    sel, _ = unpack_bits(blob, off, rows, 2)
    off += (packed_nbytes(rows, 2) + 3) & ~3
    q = (sel + 1).astype(np.uint8)
    symbols = []
    for r in range(rows):
        n = cols * int(q[r]) // 8
        symbols.append(bytes(blob[off : off + n]))
        off += n
    blocks = cols // 32
    sq_rows = int(np.count_nonzero(q < 4))
    sq4_rows = rows - sq_rows
    bsel, off = unpack_bits(blob, off, sq_rows * blocks, 1) if sq_rows else (np.empty(0, np.uint8), off)
    ssc, off = unpack_bits(blob, off, sq_rows * 8, 2) if sq_rows else (np.empty(0, np.uint8), off)
    spal, off = unpack_bits(blob, off, sq_rows * 8, 5) if sq_rows else (np.empty(0, np.uint8), off)
    native = np.frombuffer(blob, dtype=np.uint8, count=sq4_rows * blocks, offset=off).reshape(sq4_rows, blocks).copy()
    off += native.size
    if off != len(blob):
        raise ValueError("MXFP4-SQ payload size mismatch")
    return Mxfp4SqTensor((rows, cols), base, q, symbols, bsel.reshape(sq_rows, blocks), ssc.reshape(sq_rows, 8),
                         spal.reshape(sq_rows, 8), native)


def to_mxfp4(t: Mxfp4SqTensor) -> MxTensor:
    if not t.is_native:
        raise NotImplementedError("only all-SQ4 MXFP4-SQ tensors expand to native MXFP4 here")
    rows, cols = t.shape
    values = np.frombuffer(b"".join(t.row_symbols), dtype=np.uint8).reshape(rows, cols // 2).copy()
    return MxTensor(MXFP4_DTYPE, (rows, cols), values, np.asarray(t.native_scales, dtype=np.uint8))


def dequantize_mxfp4sq(t: Mxfp4SqTensor) -> np.ndarray:
    from .mx import dequantize_mx
    return dequantize_mx(to_mxfp4(t))
