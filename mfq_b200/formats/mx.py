"""OCP microscaling payloads: MXFP4 (E2M1 + E8M0 per 1x32) and MXFP8 (E4M3 + E8M0).

Blob (``"MXT1"`` header of 56 bytes, then values, then scales; layout parity with
``mfq/formats/mx.py:21-27,145-181`` of the reference)::

    "MXT1" u8 version=1  u8 kind (4|8)  u16 0
    u64 rows, cols, storage_rows, storage_cols, scale_rows, scale_cols
    values   MXFP4: rows x cols/2 bytes, element 2j in the low nibble
             MXFP8: rows x cols E4M3 bytes
    scales   E8M0 bytes (value 2**(e-127); 255 = NaN is rejected)
             MXFP4: rows x cols/32;  MXFP8: per 1x32, 32x32 or 128x128 block

These are also the operand formats of the block-scaled ``tcgen05.mma`` kinds
(``mxf4`` / ``mxf8f6f4``), so a payload can be uploaded without re-encoding.
"""

from __future__ import annotations

import math
import struct
from dataclasses import dataclass

import numpy as np

MXFP4_DTYPE = "MXFP4"
MXFP8_DTYPE = "MXFP8"
_HEAD = struct.Struct("<4sBBHQQQQQQ")
_MAGIC = b"MXT1"

# E2M1 code -> value (sign in bit 3)
E2M1_VALUES = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], dtype=np.float32)

__all__ = [
    "MXFP4_DTYPE", "MXFP8_DTYPE", "MxTensor", "pack_mx", "unpack_mx", "dequantize_mx",
    "E2M1_VALUES", "e8m0_to_float", "e4m3_to_float", "float_to_e4m3",
]


def e8m0_to_float(codes: np.ndarray) -> np.ndarray:
    return np.ldexp(np.float32(1.0), np.asarray(codes, dtype=np.int32) - 127).astype(np.float32)


def _e4m3_table() -> np.ndarray:
    codes = np.arange(256, dtype=np.int32)
    sign = np.where(codes & 0x80, -1.0, 1.0)
    exp = (codes >> 3) & 0xF
    man = codes & 0x7
    val = np.where(exp == 0, man / 8.0 * 2.0 ** -6, (1.0 + man / 8.0) * np.exp2(exp - 7.0))
    val = np.where((codes & 0x7F) == 0x7F, np.nan, val)
    return (sign * val).astype(np.float32)


E4M3_TABLE = _e4m3_table()
_E4M3_POS = E4M3_TABLE[:127].copy()  # codes 0..126 are the finite non-negative values, ascending


def e4m3_to_float(codes: np.ndarray) -> np.ndarray:
    return E4M3_TABLE[np.asarray(codes, dtype=np.uint8)]


def float_to_e4m3(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even to finite E4M3 (saturating at +-448); returns uint8 codes."""
    x = np.asarray(x, dtype=np.float32)
    mag = np.minimum(np.abs(x), np.float32(448.0))
    hi = np.searchsorted(_E4M3_POS, mag, side="left").clip(0, 126)
    lo = np.maximum(hi - 1, 0)
    d_hi = _E4M3_POS[hi] - mag
    d_lo = mag - _E4M3_POS[lo]
    pick_lo = (d_lo < d_hi) | ((d_lo == d_hi) & ((lo & 1) == 0))
    code = np.where(pick_lo, lo, hi).astype(np.uint8)
    return code | (np.signbit(x).astype(np.uint8) << 7)


@dataclass(frozen=True)
class MxTensor:
    dtype: str
    shape: tuple[int, int]
    values: np.ndarray  # uint8 storage matrix
    scales: np.ndarray  # uint8 E8M0 matrix

    def __post_init__(self) -> None:
        _geometry(self.dtype, self.shape, tuple(self.values.shape), tuple(self.scales.shape))
        if np.any(np.asarray(self.scales).view(np.uint8) == 255):
            raise ValueError(f"{self.dtype} contains an E8M0 NaN scale")
        if self.dtype == MXFP8_DTYPE and np.any((np.asarray(self.values).view(np.uint8) & 0x7F) == 0x7F):
            raise ValueError("MXFP8 contains an E4M3 NaN code")

    @property
    def block_shape(self) -> tuple[int, int]:
        if self.dtype == MXFP4_DTYPE:
            return (1, 32)
        rows, cols = self.shape
        for blk in ((128, 128), (32, 32), (1, 32)):
            if tuple(self.scales.shape) == (math.ceil(rows / blk[0]), math.ceil(cols / blk[1])):
                return blk
        raise ValueError("unsupported MXFP8 scale geometry")


def _geometry(dtype, shape, storage, scale_shape) -> None:
    if dtype not in (MXFP4_DTYPE, MXFP8_DTYPE):
        raise ValueError(f"unsupported MX dtype {dtype}")
    rows, cols = (int(v) for v in shape)
    if rows <= 0 or cols <= 0 or cols % 32:
        raise ValueError(f"{dtype} needs a non-empty matrix whose columns divide by 32")
    if dtype == MXFP4_DTYPE:
        if storage != (rows, cols // 2) or scale_shape != (rows, cols // 32):
            raise ValueError("MXFP4 storage/scale shape mismatch")
        return
    ok = {((rows + 31) // 32, cols // 32), (rows, cols // 32)}
    if cols % 128 == 0:
        ok.add(((rows + 127) // 128, cols // 128))
    if storage != (rows, cols) or tuple(scale_shape) not in ok:
        raise ValueError("MXFP8 storage/scale shape mismatch")


def pack_mx(t: MxTensor) -> bytes:
    v = np.ascontiguousarray(t.values).view(np.uint8)
    s = np.ascontiguousarray(t.scales).view(np.uint8)
    kind = 4 if t.dtype == MXFP4_DTYPE else 8
    return _HEAD.pack(_MAGIC, 1, kind, 0, *t.shape, *v.shape, *s.shape) + v.tobytes() + s.tobytes()


def unpack_mx(dtype: str, blob) -> MxTensor:
    if len(blob) < _HEAD.size:
        raise ValueError("truncated MX header")
    magic, version, kind, reserved, rows, cols, srows, scols, crow, ccol = _HEAD.unpack_from(blob, 0)
    want = 4 if dtype == MXFP4_DTYPE else 8
    if magic != _MAGIC or version != 1 or kind != want or reserved:
        raise ValueError(f"invalid {dtype} payload header")
    _geometry(dtype, (rows, cols), (srows, scols), (crow, ccol))
    nv, ns = srows * scols, crow * ccol
    if len(blob) != _HEAD.size + nv + ns:
        raise ValueError(f"{dtype} payload size mismatch")
    values = np.frombuffer(blob, dtype=np.uint8, count=nv, offset=_HEAD.size).reshape(srows, scols).copy()
    scales = np.frombuffer(blob, dtype=np.uint8, count=ns, offset=_HEAD.size + nv).reshape(crow, ccol).copy()
    return MxTensor(dtype, (rows, cols), values, scales)


def dequantize_mx(t: MxTensor) -> np.ndarray:
    rows, cols = t.shape
    if t.dtype == MXFP4_DTYPE:
        v = np.asarray(t.values, dtype=np.uint8)
        nib = np.empty((rows, cols), dtype=np.uint8)
        nib[:, 0::2] = v & 0x0F
        nib[:, 1::2] = v >> 4
        mag = E2M1_VALUES[nib & 7]
        val = np.where(nib & 8, -mag, mag)
        return val * np.repeat(e8m0_to_float(t.scales), 32, axis=1)
    br, bc = t.block_shape
    scale = np.repeat(np.repeat(e8m0_to_float(t.scales), br, axis=0)[:rows], bc, axis=1)[:, :cols]
    return e4m3_to_float(t.values) * scale
