"""NINT8-0: symmetric 8-bit blocks, byte-identical to GGML ``Q8_0`` under an MFQ dtype label.

Payload: ``"NI80"  i32 axis  i32 neuron_len  u32 ndim  ndim x i64 shape  u32 out  u32 groups`` followed by
``out * groups`` blocks of 34 bytes: one fp16 scale and 32 signed bytes, ``w = scale * q``.  Quantization is the
deterministic Q8_0 rule ``scale = amax / 127``, ``q = round(w / scale)``.  Layout parity:
``mfq/formats/nint8_zero.py:1-12,77-130`` of the reference.
"""

from __future__ import annotations

import struct
from dataclasses import dataclass

import numpy as np

NINT8_ZERO_DTYPE = "NINT8-0"
BLOCK = 32
_MAGIC = b"NI80"
_HEAD = struct.Struct("<4siiI")


@dataclass
class Nint8ZeroTensor:
    shape: tuple[int, ...]
    axis: int
    scale: np.ndarray  # [out, groups] fp16, non-negative
    q: np.ndarray  # [out, groups, 32] int8

    @property
    def neuron_len(self) -> int:
        return self.q.shape[1] * BLOCK


def quantize_nint8_zero(weight, axis: int = 0) -> Nint8ZeroTensor:
    w = np.asarray(weight, dtype=np.float32)
    rows = np.moveaxis(w, axis, 0).reshape(w.shape[axis], -1)
    if rows.shape[1] % BLOCK:
        raise ValueError("NINT8-0 needs a row length that is a multiple of 32")
    blocks = rows.reshape(rows.shape[0], -1, BLOCK)
    d = np.abs(blocks).max(-1) / 127.0
    inv = np.where(d > 0, 1.0 / np.where(d > 0, d, 1.0), 0.0).astype(np.float32)
    q = np.rint(blocks * inv[..., None]).clip(-127, 127).astype(np.int8)
    return Nint8ZeroTensor(tuple(w.shape), axis, d.astype(np.float16), q)


def dequantize_nint8_zero(t: Nint8ZeroTensor) -> np.ndarray:
    rows = (t.q.astype(np.float32) * t.scale.astype(np.float32)[..., None]).reshape(t.q.shape[0], -1)
    shape, axis = tuple(t.shape), t.axis
    moved = (shape[axis],) + shape[:axis] + shape[axis + 1 :]
    return np.moveaxis(rows.reshape(moved), 0, axis)


def pack_nint8_zero(t: Nint8ZeroTensor) -> bytes:
    out, groups = t.scale.shape
    blocks = np.empty((out, groups, 2 + BLOCK), dtype=np.uint8)
    blocks[..., :2] = np.ascontiguousarray(t.scale, dtype="<f2").view(np.uint8).reshape(out, groups, 2)
    blocks[..., 2:] = t.q.view(np.uint8)
    head = _HEAD.pack(_MAGIC, t.axis, t.neuron_len, len(t.shape)) + struct.pack(f"<{len(t.shape)}q", *t.shape)
    return head + struct.pack("<II", out, groups) + blocks.tobytes()


def unpack_nint8_zero(blob) -> Nint8ZeroTensor:
    magic, axis, neuron_len, ndim = _HEAD.unpack_from(blob, 0)
    if magic != _MAGIC:
        raise ValueError(f"invalid NINT8-0 magic: {magic!r}")
    off = _HEAD.size
    shape = tuple(struct.unpack_from(f"<{ndim}q", blob, off))
    off += 8 * ndim
    out, groups = struct.unpack_from("<II", blob, off)
    off += 8
    if groups * BLOCK != neuron_len or off + out * groups * (2 + BLOCK) != len(blob):
        raise ValueError("NINT8-0 payload size does not match its header")
    blocks = np.frombuffer(blob, dtype=np.uint8, count=out * groups * (2 + BLOCK), offset=off).reshape(out, groups, 2 + BLOCK)
    scale = np.ascontiguousarray(blocks[..., :2]).view("<f2").reshape(out, groups).copy()
    if not np.isfinite(scale).all() or np.signbit(scale).any():
        raise ValueError("NINT8-0 scales must be finite and non-negative")
    return Nint8ZeroTensor(shape, axis, scale, np.ascontiguousarray(blocks[..., 2:]).view(np.int8).copy())
