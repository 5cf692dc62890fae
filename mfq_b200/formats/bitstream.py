"""LSB-first bitstreams used by every packed MFQ payload.

Value ``i`` of width ``b`` occupies bits ``[i*b, (i+1)*b)`` of the stream; bit 0
of byte 0 comes first.  This is the convention of the reference container
(``mfq/formats/io.py:321-378`` for NINT payloads, ``mfq/formats/nvq.py:760-789``
for NVQ payloads); both reduce to the same bit order, so one generic
implementation serves all families here.
"""

from __future__ import annotations

import numpy as np

__all__ = ["pack_bits", "unpack_bits", "packed_nbytes"]


def packed_nbytes(count: int, bits: int) -> int:
    return (int(count) * int(bits) + 7) // 8


def pack_bits(values: np.ndarray, bits: int) -> bytes:
    """Pack unsigned integers (< 2**bits) into an LSB-first bitstream."""
    if not 1 <= bits <= 16:
        raise ValueError(f"unsupported packed width: {bits}")
    flat = np.ascontiguousarray(values).reshape(-1)
    if flat.size and int(flat.max()) >> bits:
        raise ValueError(f"value exceeds {bits}-bit packed width")
    if bits == 8:
        return flat.astype(np.uint8, copy=False).tobytes()
    if bits == 16:
        return flat.astype("<u2", copy=False).tobytes()
    if bits == 4:
        u = flat.astype(np.uint8, copy=False)
        if u.size & 1:
            u = np.append(u, np.uint8(0))
        return (u[0::2] | (u[1::2] << 4)).astype(np.uint8).tobytes()
    wide = flat.astype(np.uint16, copy=False)
    # Chunk to bound the (n, bits) temporary for very large tensors.
    out = bytearray()
    step = 1 << 22  # multiple of 8 values, so every chunk ends on a byte boundary
    for start in range(0, wide.size, step):
        part = wide[start : start + step]
        lanes = ((part[:, None] >> np.arange(bits, dtype=np.uint16)[None, :]) & 1).astype(np.uint8)
        out += np.packbits(lanes.reshape(-1), bitorder="little").tobytes()
    return bytes(out)


def unpack_bits(blob, offset: int, count: int, bits: int) -> tuple[np.ndarray, int]:
    """Inverse of :func:`pack_bits`; returns ``(values, next_offset)``."""
    if not 1 <= bits <= 16:
        raise ValueError(f"unsupported packed width: {bits}")
    nbytes = packed_nbytes(count, bits)
    if offset + nbytes > len(blob):
        raise ValueError("truncated bitstream")
    raw = np.frombuffer(blob, dtype=np.uint8, count=nbytes, offset=offset)
    if bits == 8:
        return raw.copy(), offset + nbytes
    if bits == 16:
        return raw.view("<u2").astype(np.uint16), offset + nbytes
    if bits == 4:
        both = np.empty(nbytes * 2, dtype=np.uint8)
        both[0::2] = raw & 0x0F
        both[1::2] = raw >> 4
        return both[:count].copy(), offset + nbytes
    out_dtype = np.uint8 if bits <= 8 else np.uint16
    result = np.empty(count, dtype=out_dtype)
    step = 1 << 22
    weights = (1 << np.arange(bits, dtype=np.uint32)).astype(np.uint32)
    for start in range(0, count, step):
        n = min(step, count - start)
        b0 = start * bits // 8  # start is a multiple of 8 values → byte aligned
        b1 = b0 + packed_nbytes(n, bits)
        lanes = np.unpackbits(raw[b0:b1], bitorder="little")[: n * bits].reshape(n, bits)
        result[start : start + n] = (lanes.astype(np.uint32) @ weights).astype(out_dtype)
    return result, offset + nbytes
