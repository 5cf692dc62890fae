"""Neuron-anchored ternary format (about 1.9 bits per weight): ``w = anchor[row] * sub[row, group] * t`` with
``t in {-1, 0, +1}``, an f16 anchor per output neuron and a k-bit integer multiplier per group of weights.

Blob (byte-compatible with ``mfq/formats/ternary.py`` of the reference): ``"NTQ\\x01"``, u8 sub_bits, u16 groupsize,
i32 axis, i32 neuron_len, u32 rank, rank x i64 shape, u32 rows, rows x f16 anchors, the k-bit multipliers as a
little-endian bit stream, then the symbols ``t + 1`` five to a byte in base 3 (first symbol least significant).
The quantizer is ours: per group it tries every multiplier, thresholds the weights at half a step and keeps the
multiplier with the least squared error, then refits the row anchor by least squares and repeats.
"""

from __future__ import annotations

import math
import struct
from dataclasses import dataclass

import numpy as np

MAGIC = b"NTQ\x01"
_HEAD = struct.Struct("<4sBHiiI")
_POW3 = np.array([1, 3, 9, 27, 81], dtype=np.uint16)


@dataclass
class TernaryTensor:
    shape: tuple[int, ...]
    axis: int
    groupsize: int
    sub_bits: int
    anchors: np.ndarray  # [rows] float32 (f16-representable)
    sub: np.ndarray  # [rows, groups] uint8
    trits: np.ndarray  # [rows, neuron_len] uint8 in {0, 1, 2}

    @property
    def neuron_len(self) -> int:
        return int(self.trits.shape[1])

    @property
    def bits_per_weight(self) -> float:
        rows, n = self.trits.shape
        groups = math.ceil(n / self.groupsize)
        return 8.0 * (rows * 2 + (rows * groups * self.sub_bits + 7) // 8 + (rows * n + 4) // 5) / (rows * n)


def _bits_pack(values: np.ndarray, bits: int) -> bytes:
    v = np.ascontiguousarray(values, dtype=np.uint16).reshape(-1)
    planes = ((v[:, None] >> np.arange(bits, dtype=np.uint16)) & 1).astype(np.uint8)
    return np.packbits(planes.reshape(-1), bitorder="little").tobytes()


def _bits_unpack(buf: bytes, off: int, count: int, bits: int) -> tuple[np.ndarray, int]:
    n = (count * bits + 7) // 8
    planes = np.unpackbits(np.frombuffer(buf, dtype=np.uint8, count=n, offset=off), bitorder="little")[: count * bits]
    vals = (planes.reshape(count, bits).astype(np.uint16) << np.arange(bits, dtype=np.uint16)).sum(1)
    return vals.astype(np.uint8), off + n


def pack(t: TernaryTensor) -> bytes:
    rows, n = t.trits.shape
    sym = np.ascontiguousarray(t.trits, dtype=np.uint8).reshape(-1)
    sym = np.pad(sym, (0, (-sym.size) % 5)).reshape(-1, 5).astype(np.uint16)
    return b"".join([
        _HEAD.pack(MAGIC, t.sub_bits, t.groupsize, t.axis, n, len(t.shape)), struct.pack(f"<{len(t.shape)}q", *t.shape),
        struct.pack("<I", rows), np.asarray(t.anchors, dtype=np.float16).tobytes(), _bits_pack(t.sub, t.sub_bits),
        (sym * _POW3).sum(1).astype(np.uint8).tobytes()])


def unpack(buf: bytes) -> TernaryTensor:
    magic, sub_bits, groupsize, axis, n, rank = _HEAD.unpack_from(buf)
    if magic != MAGIC:
        raise ValueError("not a ternary blob")
    off = _HEAD.size
    shape = struct.unpack_from(f"<{rank}q", buf, off)
    off += 8 * rank
    rows = struct.unpack_from("<I", buf, off)[0]
    off += 4
    anchors = np.frombuffer(buf, dtype=np.float16, count=rows, offset=off).astype(np.float32)
    off += 2 * rows
    groups = math.ceil(n / groupsize)
    sub, off = _bits_unpack(buf, off, rows * groups, sub_bits)
    nbytes = (rows * n + 4) // 5
    packed = np.frombuffer(buf, dtype=np.uint8, count=nbytes, offset=off).astype(np.uint16)
    if packed.size and packed.max() > 242:
        raise ValueError("invalid base-3 byte")
    trits = np.stack([(packed // p) % 3 for p in _POW3], 1).reshape(-1)[: rows * n].astype(np.uint8)
    if off + nbytes != len(buf):
        raise ValueError("trailing bytes after the ternary payload")
    return TernaryTensor(tuple(shape), axis, groupsize, sub_bits, anchors, sub.reshape(rows, groups), trits.reshape(rows, n))


def dequantize(t: TernaryTensor) -> np.ndarray:
    scale = np.repeat(t.anchors[:, None] * t.sub.astype(np.float32), t.groupsize, axis=1)[:, : t.neuron_len]
    rows = (t.trits.astype(np.float32) - 1.0) * scale
    moved = (t.shape[t.axis],) + t.shape[: t.axis] + t.shape[t.axis + 1 :]
    return np.moveaxis(rows.reshape(moved), 0, t.axis)


def quantize(w: np.ndarray, groupsize: int = 24, sub_bits: int = 3, axis: int = 0, iters: int = 3) -> TernaryTensor:
    w = np.asarray(w, dtype=np.float32)
    rows = np.moveaxis(w, axis, 0).reshape(w.shape[axis], -1)
    r, n = rows.shape
    groups = math.ceil(n / groupsize)
    pad = groups * groupsize - n
    x = np.pad(rows, ((0, 0), (0, pad))).reshape(r, groups, groupsize)
    live = np.pad(np.ones((r, n), bool), ((0, 0), (0, pad))).reshape(r, groups, groupsize)
    qmax = (1 << sub_bits) - 1
    # a ternary code with step s represents |x| ~ s best when s ~ mean |x| of the kept weights; start the largest
    # multiplier near the strongest group's step
    step = np.abs(x).mean(-1).max(-1) * 1.4 + 1e-12
    anchors = (step / qmax).astype(np.float16).astype(np.float32)
    anchors[anchors == 0] = np.float32(np.finfo(np.float16).tiny)
    cands = np.arange(qmax + 1, dtype=np.float32)
    for _ in range(iters):
        s = anchors[:, None, None, None] * cands[None, None, :, None]  # [r, 1, q, 1]
        xe = x[:, :, None, :]
        code = np.where(np.abs(xe) > 0.5 * s, np.sign(xe), 0.0) * (s > 0)
        err = (((xe - code * s) ** 2) * live[:, :, None, :]).sum(-1)  # [r, groups, q]
        sub = err.argmin(-1)
        sel = np.take_along_axis(code, sub[:, :, None, None], 2)[:, :, 0, :]
        basis = sel * sub[:, :, None].astype(np.float32)  # w ~ anchor * basis
        num, den = (basis * x).sum((1, 2)), (basis * basis).sum((1, 2))
        refit = np.where(den > 0, num / np.maximum(den, 1e-30), anchors)
        anchors = np.maximum(refit, np.finfo(np.float16).tiny).astype(np.float16).astype(np.float32)
    trits = (sel + 1).astype(np.uint8).reshape(r, -1)[:, :n]
    return TernaryTensor(tuple(w.shape), axis, groupsize, sub_bits, anchors, sub.astype(np.uint8), trits)
