"""Dense tensor payloads: ``u32 ndim, i64 shape[ndim], raw little-endian data``.

bf16 and E4M3 have no NumPy dtype, so they travel as ``uint16`` / ``uint8`` bit
patterns wrapped in thin ndarray subclasses that remember what the bits mean
(layout parity: ``mfq/formats/io.py:873-925`` of the reference).
"""

from __future__ import annotations

import struct

import numpy as np


class Bf16Array(np.ndarray):
    """``uint16`` array whose elements are bfloat16 bit patterns."""


class Fp8E4M3Array(np.ndarray):
    """``uint8`` array whose elements are E4M3 bit patterns."""


DENSE_DTYPES = {
    "BF16": np.dtype("<u2"), "F8_E4M3": np.dtype("u1"), "F16": np.dtype("<f2"), "F32": np.dtype("<f4"),
    "I32": np.dtype("<i4"), "I64": np.dtype("<i8"), "U8": np.dtype("u1"), "I8": np.dtype("i1"),
}
_BY_NUMPY = {np.dtype("float16"): "F16", np.dtype("float32"): "F32", np.dtype("int32"): "I32",
             np.dtype("int64"): "I64", np.dtype("uint8"): "U8", np.dtype("int8"): "I8"}


def to_bf16(x: np.ndarray) -> Bf16Array:
    """float32 -> bfloat16 bits, round-to-nearest-even."""
    bits = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    rounded = ((bits + 0x7FFF + ((bits >> 16) & 1)) >> 16).astype(np.uint16)
    return rounded.view(Bf16Array)


def from_bf16(x: np.ndarray) -> np.ndarray:
    return (np.asarray(x).view(np.uint16).astype(np.uint32) << 16).view(np.float32)


def pack_dense(t: np.ndarray) -> tuple[str, bytes]:
    if isinstance(t, Bf16Array):
        name = "BF16"
    elif isinstance(t, Fp8E4M3Array):
        name = "F8_E4M3"
    else:
        name = _BY_NUMPY.get(np.asarray(t).dtype)
        if name is None:
            raise ValueError(f"unsupported dense dtype {np.asarray(t).dtype}")
    a = np.ascontiguousarray(t)
    return name, struct.pack("<I", a.ndim) + struct.pack(f"<{a.ndim}q", *a.shape) + a.tobytes()


def unpack_dense(dtype: str, blob) -> np.ndarray:
    (ndim,) = struct.unpack_from("<I", blob, 0)
    shape = struct.unpack_from(f"<{ndim}q", blob, 4)
    a = np.frombuffer(blob, dtype=DENSE_DTYPES[dtype], offset=4 + 8 * ndim).reshape(shape).copy()
    if dtype == "BF16":
        return a.view(Bf16Array)
    if dtype == "F8_E4M3":
        return a.view(Fp8E4M3Array)
    return a
