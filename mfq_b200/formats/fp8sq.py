"""FP8-128SQ / MXFP8-SQ: E4M3 matrices with block scales and per-row scalar palettes.

Every row stores its E4M3 codes either raw (SQ8) or as ``q``-bit symbols
(SQ1..SQ7) into one tensor-wide palette of ``2**q`` legal E4M3 codes.  Scales are
one E8M0 byte per 1x32 / 32x32 / 128x128 block (``MXFP8-SQ``, magic ``M8SQ``) or one
BF16/F16/F32 multiplier per 128x128 block (``FP8-128SQ``, magic ``F8SQ``).

*Block-FP8 as served by this framework is the all-SQ8 + F32-scale case*: the
payload is exactly the E4M3 byte matrix followed by the fp32 scale grid, which is
what the tensor-core GEMM consumes with no decode step.

Blob (44-byte header; parity with ``mfq/formats/fp8_sq.py:36-56,262-300`` of the
reference)::

    magic[4] u8 version=1 u8 scale_kind(1 E8M0,2 BF16,3 F16,4 F32) u8 flags=0 u8 0
    u16 block_rows, block_cols   u64 rows, cols, scale_rows, scale_cols
    row selectors  rows x 3 bit (q-1), zero padded to a multiple of 4 bytes
    palettes       256 bytes; palette of SQq at [2**q - 2, 2**(q+1) - 2), last 2 bytes 0
    symbols        per row ceil(cols*q/8) bytes (byte aligned per row)
    scales         scale_rows x scale_cols items
"""

from __future__ import annotations

import struct
from dataclasses import dataclass, field

import numpy as np

from .bitstream import pack_bits, unpack_bits, packed_nbytes
from .mx import e4m3_to_float, e8m0_to_float

FP8_128SQ_DTYPE = "FP8-128SQ"
MXFP8_SQ_DTYPE = "MXFP8-SQ"
_HEAD = struct.Struct("<4sBBBBHHQQQQ")
_MAGIC = {FP8_128SQ_DTYPE: b"F8SQ", MXFP8_SQ_DTYPE: b"M8SQ"}
_SCALE_KINDS = {"F8_E8M0": 1, "BF16": 2, "F16": 3, "F32": 4}
_SCALE_NAMES = {v: k for k, v in _SCALE_KINDS.items()}
_SCALE_SIZE = {"F8_E8M0": 1, "BF16": 2, "F16": 2, "F32": 4}
_PALETTE_BYTES = 256

__all__ = [
    "FP8_128SQ_DTYPE", "MXFP8_SQ_DTYPE", "Fp8SqTensor", "pack_fp8sq", "unpack_fp8sq", "dequantize_fp8sq",
    "palette_slice", "block_fp8_tensor",
]


def default_palettes() -> np.ndarray:
    """Placeholder palette region for tensors without SQ1..SQ7 rows: codes ``0..2**q-1`` per width.

    Readers insist on duplicate-free palettes even when no row uses them.
    """
    pal = np.zeros(_PALETTE_BYTES, dtype=np.uint8)
    for q in range(1, 8):
        pal[(1 << q) - 2 : (1 << (q + 1)) - 2] = np.arange(1 << q, dtype=np.uint8)
    pal[253] = 0x80  # 0x7F is the E4M3 NaN code; -0 takes its place in the 7-bit palette
    return pal


def palette_slice(q: int) -> slice:
    if not 1 <= q <= 7:
        raise ValueError("palettes exist for SQ1..SQ7 only")
    return slice((1 << q) - 2, (1 << (q + 1)) - 2)


@dataclass
class Fp8SqTensor:
    dtype: str
    shape: tuple[int, int]
    codes: np.ndarray  # [rows, cols] uint8 E4M3 codes (already palette-expanded)
    scales: np.ndarray  # float32 multipliers, or uint8 E8M0 codes for MXFP8-SQ
    block_shape: tuple[int, int] = (128, 128)
    scale_dtype: str = "F32"
    row_q_bits: np.ndarray | None = None  # [rows] in 1..8; None = all SQ8
    palettes: np.ndarray = field(default_factory=lambda: default_palettes())

    def q_widths(self) -> np.ndarray:
        if self.row_q_bits is None:
            return np.full(self.shape[0], 8, dtype=np.uint8)
        return np.asarray(self.row_q_bits, dtype=np.uint8)

    @property
    def scale_shape(self) -> tuple[int, int]:
        (r, c), (br, bc) = self.shape, self.block_shape
        return ((r + br - 1) // br, (c + bc - 1) // bc)


def _check(t: Fp8SqTensor) -> None:
    rows, cols = t.shape
    if t.dtype not in _MAGIC or rows <= 0 or cols <= 0:
        raise ValueError("invalid FP8-SQ tensor")
    if tuple(np.asarray(t.scales).shape) != t.scale_shape:
        raise ValueError(f"FP8-SQ scale shape {np.asarray(t.scales).shape} != {t.scale_shape}")
    if t.dtype == FP8_128SQ_DTYPE:
        if t.block_shape != (128, 128) or t.scale_dtype not in ("BF16", "F16", "F32"):
            raise ValueError("FP8-128SQ needs 128x128 blocks with BF16/F16/F32 multipliers")
        s = np.asarray(t.scales, dtype=np.float32)
        if not np.isfinite(s).all() or np.any(s <= 0):
            raise ValueError("FP8-128SQ multipliers must be positive and finite")
    else:
        if t.scale_dtype != "F8_E8M0" or t.block_shape not in ((1, 32), (32, 32), (128, 128)) or cols % t.block_shape[1]:
            raise ValueError("MXFP8-SQ needs E8M0 scales over complete 1x32/32x32/128x128 blocks")
        if np.any(np.asarray(t.scales) == 255):
            raise ValueError("MXFP8-SQ contains an E8M0 NaN scale")
    if np.any((np.asarray(t.codes, dtype=np.uint8) & 0x7F) == 0x7F):
        raise ValueError("FP8-SQ contains an E4M3 NaN code")
    pal = np.asarray(t.palettes, dtype=np.uint8).reshape(-1)
    if pal.size != _PALETTE_BYTES or np.any(pal[254:]) or np.any((pal[:254] & 0x7F) == 0x7F):
        raise ValueError("invalid FP8-SQ palette region")
    for q in range(1, 8):
        p = pal[palette_slice(q)]
        if np.unique(p).size != p.size:
            raise ValueError(f"SQ{q} palette holds duplicate codes")


def _scale_bytes(t: Fp8SqTensor) -> bytes:
    s = np.asarray(t.scales)
    if t.scale_dtype == "F8_E8M0":
        return s.astype(np.uint8).tobytes()
    s = s.astype(np.float32)
    if t.scale_dtype == "F32":
        return s.astype("<f4").tobytes()
    if t.scale_dtype == "F16":
        return s.astype("<f2").tobytes()
    bits = s.view(np.uint32)
    rounded = (bits + 0x7FFF + ((bits >> 16) & 1)) >> 16  # round-to-nearest-even to bf16
    return rounded.astype("<u2").tobytes()


def pack_fp8sq(t: Fp8SqTensor) -> bytes:
    _check(t)
    rows, cols = t.shape
    qw = t.q_widths()
    sel = pack_bits(qw - 1, 3)
    sel += b"\0" * (((len(sel) + 3) & ~3) - len(sel))
    pal = np.asarray(t.palettes, dtype=np.uint8).reshape(-1)
    codes = np.ascontiguousarray(t.codes, dtype=np.uint8)
    head = _HEAD.pack(_MAGIC[t.dtype], 1, _SCALE_KINDS[t.scale_dtype], 0, 0, *t.block_shape, rows, cols, *t.scale_shape)
    if np.all(qw == 8):
        body = codes.tobytes()
    else:
        inverse = {}
        for q in range(1, 8):
            lut = np.full(256, -1, dtype=np.int16)
            p = pal[palette_slice(q)]
            lut[p] = np.arange(p.size)
            inverse[q] = lut
        chunks = []
        for r in range(rows):
            q = int(qw[r])
            if q == 8:
                chunks.append(codes[r].tobytes())
                continue
            sym = inverse[q][codes[r]]
            if sym.min() < 0:
                raise ValueError(f"row {r} uses a code outside its SQ{q} palette")
            chunks.append(pack_bits(sym.astype(np.uint8), q))
        body = b"".join(chunks)
    return b"".join([head, sel, pal.tobytes(), body, _scale_bytes(t)])


def unpack_fp8sq(dtype: str, blob) -> Fp8SqTensor:
    if dtype not in _MAGIC or len(blob) < _HEAD.size:
        raise ValueError("invalid FP8-SQ payload")
    magic, version, kind, flags, reserved, br, bc, rows, cols, srows, scols = _HEAD.unpack_from(blob, 0)
    if magic != _MAGIC[dtype] or version != 1 or flags or reserved or kind not in _SCALE_NAMES:
        raise ValueError(f"invalid {dtype} header")
    scale_dtype = _SCALE_NAMES[kind]
    off = _HEAD.size
    sel, _ = unpack_bits(blob, off, rows, 3)
    off += (packed_nbytes(rows, 3) + 3) & ~3
    pal = np.frombuffer(blob, dtype=np.uint8, count=_PALETTE_BYTES, offset=off).copy()
    off += _PALETTE_BYTES
    qw = (sel + 1).astype(np.uint8)
    codes = np.empty((rows, cols), dtype=np.uint8)
    if np.all(qw == 8):
        codes[:] = np.frombuffer(blob, dtype=np.uint8, count=rows * cols, offset=off).reshape(rows, cols)
        off += rows * cols
    else:
        for r in range(rows):
            q = int(qw[r])
            if q == 8:
                codes[r] = np.frombuffer(blob, dtype=np.uint8, count=cols, offset=off)
                off += cols
            else:
                sym, off = unpack_bits(blob, off, cols, q)
                codes[r] = pal[palette_slice(q)][sym]
    n = srows * scols
    raw = np.frombuffer(blob, dtype=np.uint8, count=n * _SCALE_SIZE[scale_dtype], offset=off)
    off += raw.size
    if off != len(blob):
        raise ValueError(f"{dtype} payload size mismatch")
    if scale_dtype == "F8_E8M0":
        scales = raw.reshape(srows, scols).copy()
    elif scale_dtype == "F32":
        scales = raw.view("<f4").reshape(srows, scols).astype(np.float32)
    elif scale_dtype == "F16":
        scales = raw.view("<f2").reshape(srows, scols).astype(np.float32)
    else:
        scales = (raw.view("<u2").astype(np.uint32) << 16).view(np.float32).reshape(srows, scols).copy()
    t = Fp8SqTensor(dtype, (rows, cols), codes, scales, (br, bc), scale_dtype, qw, pal)
    _check(t)
    return t


def dequantize_fp8sq(t: Fp8SqTensor) -> np.ndarray:
    rows, cols = t.shape
    br, bc = t.block_shape
    s = e8m0_to_float(t.scales) if t.scale_dtype == "F8_E8M0" else np.asarray(t.scales, dtype=np.float32)
    full = np.repeat(np.repeat(s, br, axis=0)[:rows], bc, axis=1)[:, :cols]
    return e4m3_to_float(t.codes) * full


def block_fp8_tensor(codes: np.ndarray, scales: np.ndarray) -> Fp8SqTensor:
    """Wrap a raw E4M3 matrix + fp32 128x128 multipliers as an all-SQ8 FP8-128SQ tensor."""
    codes = np.ascontiguousarray(codes, dtype=np.uint8)
    return Fp8SqTensor(FP8_128SQ_DTYPE, tuple(codes.shape), codes, np.asarray(scales, dtype=np.float32))
