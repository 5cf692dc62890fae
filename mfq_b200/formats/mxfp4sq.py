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

Decoding a ``q < 4`` row (``mfq/kernels/cuda/mxfp4_sq.cu:43-99`` of the reference).  A block of
32 symbols names one of the row's eight STATES with three bits: the block's selector bit is
bit 2, and bits 0-1 are the XOR of the low two bits of the block's symbols (for ``q = 1`` the
XOR of the 16 two-bit pairs of neighbouring symbols) -- two bits of side information that cost
no storage; the encoder steers them by nudging a symbol.  State ``s`` gives the block its
E8M0 exponent ``matrix_scale_base + state_scale[s]`` and its palette ``state_palette[s]``, one
of 32 catalogue palettes for that ``q``; a palette maps a symbol to an E2M1 nibble.  So every
row expands to legal native MXFP4 (:func:`to_mxfp4`), which the tensor-core MXFP4 path runs.

The catalogue: a palette is a ``2**q``-subset of the 15 distinct E2M1 values in ascending
order; the subsets are numbered in lexicographic order of their positions and 32 numbers per
``q`` are fixed by the format (``mfq/quantize/mxfp4_sq.py:47-153``).
"""

from __future__ import annotations

import struct
from dataclasses import dataclass

import numpy as np

from .bitstream import pack_bits, unpack_bits, packed_nbytes
from .mx import E2M1_VALUES, MXFP4_DTYPE, MxTensor, e8m0_to_float

import itertools

MXFP4_SQ_DTYPE = "MXFP4-SQ"
# E2M1 nibbles of the 15 distinct values in ascending order: -6 .. -0.5, 0, 0.5 .. 6
ORDERED_NIBBLES = np.array([0xF, 0xE, 0xD, 0xC, 0xB, 0xA, 0x9, 0x0, 0x1, 0x2, 0x3, 0x4, 0x5, 0x6, 0x7], dtype=np.uint8)
_CATALOGUE_IDS = {
    1: (12, 26, 38, 11, 13, 58, 22, 48, 25, 23, 67, 21, 37, 24, 75, 20, 8, 59, 68, 9, 76, 7, 19, 36, 46, 55, 63, 70, 35, 47, 56, 45),
    2: (120, 127, 187, 504, 512, 518, 547, 548, 558, 562, 592, 767, 806, 833, 966, 967, 192, 1112, 971, 802, 559, 240, 112,
        226, 232, 182, 188, 121, 505, 848, 0, 1),
    3: (499, 2407, 523, 5738, 1196, 2001, 5497, 4705, 1087, 2400, 2402, 1077, 1078, 4116, 5503, 2002, 3726, 2010, 5498, 4117,
        5552, 4706, 500, 1483, 3717, 3727, 1478, 4818, 5811, 2003, 2989, 2035),
}


def _catalogue(q: int) -> np.ndarray:
    """[32, 2**q] E2M1 nibbles: palette ``i`` is the ``_CATALOGUE_IDS[q][i]``-th ``2**q``-subset of the ordered values."""
    want = {cid: slot for slot, cid in enumerate(_CATALOGUE_IDS[q])}
    out = np.zeros((32, 1 << q), dtype=np.uint8)
    last = max(want)
    for number, positions in enumerate(itertools.combinations(range(15), 1 << q)):
        slot = want.get(number)
        if slot is not None:
            out[slot] = ORDERED_NIBBLES[list(positions)]
        if number >= last:
            break
    out.setflags(write=False)
    return out


PALETTES = {q: _catalogue(q) for q in (1, 2, 3)}


def unpack_symbols(stream: bytes, cols: int, q: int) -> np.ndarray:
    """One row's symbol stream -> [cols] uint8 (LSB first)."""
    return unpack_bits(stream, 0, cols, q)[0].astype(np.uint8)


def block_tags(symbols: np.ndarray, q: int) -> np.ndarray:
    """``symbols [..., blocks, 32]`` -> the two tag bits every block carries in its symbols."""
    s = np.asarray(symbols, dtype=np.uint8)
    if q == 1:
        return np.bitwise_xor.reduce(s[..., 0::2], axis=-1) | (np.bitwise_xor.reduce(s[..., 1::2], axis=-1) << 1)
    return np.bitwise_xor.reduce(s & 3, axis=-1)
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
    """The native MXFP4 matrix every row decodes to (exactly the source for ``q = 4`` rows)."""
    rows, cols = t.shape
    blocks = cols // 32
    values = np.zeros((rows, cols // 2), dtype=np.uint8)
    scales = np.zeros((rows, blocks), dtype=np.uint8)
    q_of = np.asarray(t.row_q_bits, dtype=np.uint8)
    sq = native = 0
    for r in range(rows):
        q = int(q_of[r])
        if q == 4:
            values[r] = np.frombuffer(t.row_symbols[r], dtype=np.uint8)
            scales[r] = t.native_scales[native]
            native += 1
            continue
        sym = unpack_symbols(t.row_symbols[r], cols, q).reshape(blocks, 32)
        state = block_tags(sym, q) | (np.asarray(t.block_selectors[sq], dtype=np.uint8) << 2)
        exponent = int(t.matrix_scale_base) + np.asarray(t.state_scales[sq], dtype=np.int64)[state]
        if exponent.max() > 254:
            raise ValueError("MXFP4-SQ row decodes to an invalid E8M0 exponent")
        nib = PALETTES[q][np.asarray(t.state_palettes[sq], dtype=np.int64)[state][:, None], sym].reshape(cols)
        values[r] = nib[0::2] | (nib[1::2] << 4)
        scales[r] = exponent
        sq += 1
    return MxTensor(MXFP4_DTYPE, (rows, cols), values, scales)


def expanded(t: Mxfp4SqTensor) -> MxTensor:
    """:func:`to_mxfp4`, computed once per tensor object (loaders slice it expert by expert)."""
    cached = getattr(t, "_expanded", None)
    if cached is None:
        cached = to_mxfp4(t)
        object.__setattr__(t, "_expanded", cached)
    return cached


def dequantize_mxfp4sq(t: Mxfp4SqTensor) -> np.ndarray:
    from .mx import dequantize_mx
    return dequantize_mx(to_mxfp4(t))
