"""NEPQ: cross-expert codecs around and below one bit per weight for a stacked ``[experts, out, K]`` projection.

The experts of one projection share a POOL of up to 256 table banks.  A row (one output neuron of one expert) is coded
like its base format -- an FP16 anchor, a state per group of 24 weights, one index per 8-weight vector, for the ternary
bases a sign bit per group -- and every four consecutive groups (a super-group, 96 weights) carry one byte that names
the bank their tables come from.  The pool is paid for once per projection, so an expert can draw on far more table
capacity than a per-tensor codec could afford.

    profile   id  base     state  index  aux   bank bytes   extras
    NEPQ0-S   0   NPQ0-S   2 b    6 b    -     320          -
    NEPQ0-L   1   NPQ0-L   3 b    7 b    -     832          -
    NEPQ1-S   2   NVQ1-S   4 b    9 b    1 b   2048         -
    NEPQ1-L   3   NVQ1-L   3 b    11 b   1 b   4096         -
    NEPQ0-A   4   NEPQ0-S                                   sparse residual: one 8-vector per block of 24 vectors
    NEPQ1-A   5   NEPQ1-S                                   sparse residual: one (sometimes two) per block of 16

Reconstruction of a stored row: NPQ0 bases ``anchor * ladder[bank][state] * concat(first[bank][state][i & 7],
second[bank][state][i >> 3])``; ternary bases ``anchor * state * (table[bank][(aux)][i] -/+ delta)`` with ``delta`` 5/32
(S, two 512-entry banks picked by ``aux``) or 1/8 (L, one 2048-entry table), subtracted where ``aux`` is set.

Rotation.  With ``rotation_block`` B (a power of two dividing K) the STORED rows are the logical rows multiplied by a
fixed +-1 diagonal and an orthonormal Walsh-Hadamard transform on every B consecutive columns; a consumer either rotates
its activations the same way or calls :func:`dequantize_nepq` (``logical=True`` undoes the rotation).  The diagonal is a
function of (K, B, seed) alone (:func:`rotation_signs`).

Sparse residual (the ``-A`` profiles, always rotated).  A 1024-entry FP16 dictionary of 8-vectors; every block of 24
(16) vectors of a row adds one dictionary entry at one position -- a record ``id << position_bits | position`` -- and
NEPQ1-A marks by one bit per block which blocks add a second one (records stored compactly, in block order).

Blob layout (byte-compatible with ``mfq/formats/nepq.py:302-310,563-631`` of the reference)::

    "NEP1" u8 version=1  u8 profile  u8 4 (groups per super-group)  u8 flags (1 = rotated)
    u32 experts  u32 out  u32 K  u32 banks  u32 rotation block  u64 rotation seed
    banks x bank bytes   f16 anchors   states   indices   aux   u8 bank ids      (bit streams LSB first)
    residual profiles: "NRA1" u8 1  u8 record bits  u8 position bits  u8 flags (1 = second stream)  u32 1024
                       u32 blocks  u32 second records  u32 padding  u64 0  32 x 0
                       f16 dictionary[1024][8]   first records   [second mask, second records]   padding zeros

:func:`quantize_nepq` is this repository's encoder (the reference trains pools offline over whole models,
``mfq/quantize/nepq.py:761-881``, ``nepq_train.py``): banks trained on slices of the experts with the base format's own
table fitting, every super-group then takes the bank with the least error, anchors are refitted by least squares, the
residual dictionary is a k-means over the worst-reconstructed vectors.
"""

from __future__ import annotations

import hashlib
import math
import struct
from dataclasses import dataclass

import numpy as np

from . import npq0, nvq1
from .bitstream import pack_bits, packed_nbytes, unpack_bits

NEPQ_DTYPE = "NEPQ"
GROUP, VEC, SUPER = 24, 8, 4
DICTIONARY = 1024
_HEAD = struct.Struct("<4sBBBBIIIIIQ")
_RES_HEAD = struct.Struct("<4sBBBBIIIIQ32x")


@dataclass(frozen=True)
class NepqProfile:
    label: str
    profile_id: int
    base: str                 # "NPQ0-S" | "NPQ0-L" | "NVQ1-S" | "NVQ1-L"
    state_bits: int
    index_bits: int
    aux_bits: int
    bank_bytes: int
    residual_block: int = 0   # vectors per residual block (0: no residual)
    residual_second: bool = False

    @property
    def position_bits(self) -> int:
        return int(math.ceil(math.log2(self.residual_block))) if self.residual_block else 0

    @property
    def record_bits(self) -> int:
        return self.position_bits + 10 if self.residual_block else 0

    def geometry(self, k: int) -> tuple[int, int, int]:
        """(groups, vectors, super-groups) of a row of ``k`` weights."""
        ng = math.ceil(k / GROUP)
        return ng, k // VEC, math.ceil(ng / SUPER)

    def stream_nbytes(self, rows: int, k: int, banks: int) -> int:
        """Bytes after the 36-byte header, without the residual section."""
        ng, nv, ns = self.geometry(k)
        return (banks * self.bank_bytes + 2 * rows + packed_nbytes(rows * ng, self.state_bits) + packed_nbytes(rows * nv, self.index_bits)
                + (packed_nbytes(rows * ng, self.aux_bits) if self.aux_bits else 0) + rows * ns)


NEPQ0_S = NepqProfile("NEPQ0-S", 0, "NPQ0-S", 2, 6, 0, npq0.NPQ0_S.table_bytes)
NEPQ0_L = NepqProfile("NEPQ0-L", 1, "NPQ0-L", 3, 7, 0, npq0.NPQ0_L.table_bytes)
NEPQ1_S = NepqProfile("NEPQ1-S", 2, "NVQ1-S", 4, 9, 1, 2048)
NEPQ1_L = NepqProfile("NEPQ1-L", 3, "NVQ1-L", 3, 11, 1, 4096)
NEPQ0_A = NepqProfile("NEPQ0-A", 4, "NPQ0-S", 2, 6, 0, npq0.NPQ0_S.table_bytes, residual_block=24)
NEPQ1_A = NepqProfile("NEPQ1-A", 5, "NVQ1-S", 4, 9, 1, 2048, residual_block=16, residual_second=True)
PROFILES = {p.label: p for p in (NEPQ0_S, NEPQ0_L, NEPQ1_S, NEPQ1_L, NEPQ0_A, NEPQ1_A)}
_BY_ID = {p.profile_id: p for p in PROFILES.values()}
_NVQ1_BASE = {"NVQ1-S": nvq1.NVQ1_S, "NVQ1-L": nvq1.NVQ1_L_S3}


def profile_of(value) -> NepqProfile:
    if isinstance(value, NepqProfile):
        return value
    found = PROFILES.get(value) if isinstance(value, str) else _BY_ID.get(value)
    if found is None:
        raise ValueError(f"unknown NEPQ profile {value!r}")
    return found


# ---- rotation ------------------------------------------------------------------------------------------------------------
def rotation_signs(width: int, block: int, seed: int) -> np.ndarray:
    """The +-1 diagonal of a rotated tensor: a PCG64 stream seeded from BLAKE2b-128 of ``"h<block>:<seed>:<width>"``
    (little-endian integer), one draw of {0, 1} per column, 1 -> +1 and 0 -> -1  (``mfq/formats/nepq.py:192-199``)."""
    digest = hashlib.blake2b(f"h{int(block)}:{int(seed)}:{int(width)}".encode(), digest_size=16).digest()
    draws = np.random.default_rng(int.from_bytes(digest, "little")).integers(0, 2, size=int(width))
    return np.where(draws, 1, -1).astype(np.int8)


def hadamard_blocks(x: np.ndarray, block: int) -> np.ndarray:
    """Orthonormal Walsh-Hadamard transform (natural order) of every ``block`` consecutive entries of the last axis;
    its own inverse."""
    x = np.asarray(x, dtype=np.float32)
    y = x.reshape(-1, block).copy()
    h = 1
    while h < block:
        v = y.reshape(-1, block // (2 * h), 2, h)
        a, b = v[:, :, 0, :].copy(), v[:, :, 1, :].copy()
        v[:, :, 0, :], v[:, :, 1, :] = a + b, a - b
        h *= 2
    return (y * np.float32(1.0 / math.sqrt(block))).reshape(x.shape)


def rotate_rows(x: np.ndarray, block: int, seed: int) -> np.ndarray:
    """Logical rows -> stored rows."""
    return hadamard_blocks(np.asarray(x, dtype=np.float32) * rotation_signs(x.shape[-1], block, seed).astype(np.float32), block)


def unrotate_rows(x: np.ndarray, block: int, seed: int) -> np.ndarray:
    """Stored rows -> logical rows."""
    return hadamard_blocks(x, block) * rotation_signs(x.shape[-1], block, seed).astype(np.float32)


# ---- tensor --------------------------------------------------------------------------------------------------------------
@dataclass
class NepqResidual:
    dictionary: np.ndarray                  # [1024, 8] float32 holding FP16 values
    first: np.ndarray                       # [experts, out, blocks] uint16 records
    second_mask: np.ndarray | None = None   # [experts, out, blocks] 0/1
    second_records: np.ndarray | None = None  # [count of set mask bits] uint16, in block order
    padding: int = 0                        # zero bytes after the streams (alignment chosen by the writer)


@dataclass
class NepqTensor:
    profile: NepqProfile
    shape: tuple[int, int, int]             # (experts, out, K)
    anchors: np.ndarray                     # [experts, out] float32 holding FP16 values
    state: np.ndarray                       # [experts, out, groups] uint8
    indices: np.ndarray                     # [experts, out, vectors] uint8 / uint16
    aux: np.ndarray | None                  # [experts, out, groups] uint8 (ternary bases), else None
    bank_ids: np.ndarray                    # [experts, out, super-groups] uint8
    banks: np.ndarray                       # [banks, bank bytes] uint8: packed table sets of the base format
    rotation_block: int = 0
    rotation_seed: int = 0
    residual: NepqResidual | None = None

    @property
    def dtype(self) -> str:
        return NEPQ_DTYPE

    @property
    def rows(self) -> int:
        return int(self.shape[0]) * int(self.shape[1])

    @property
    def blocks_per_row(self) -> int:
        p = self.profile
        return math.ceil((self.shape[2] // VEC) / p.residual_block) if p.residual_block else 0

    @property
    def nbytes(self) -> int:
        return len(pack_nepq(self))

    def bits_per_weight(self) -> float:
        return 8.0 * (self.nbytes - _HEAD.size) / float(np.prod(self.shape))


def _decode_banks(p: NepqProfile, banks: np.ndarray):
    """Packed pool -> arrays indexed by bank.  NPQ0: (ladder [B, S], first [B, S, 8, 4], second [B, S, n, 4]);
    NVQ1-S: [B, 2, 512, 8]; NVQ1-L: [B, 2048, 8]."""
    rows = [bytes(r) for r in np.ascontiguousarray(banks, dtype=np.uint8)]
    if p.base.startswith("NPQ0"):
        v = npq0.VARIANTS[p.base]
        parts = [npq0.unpack_tables(v, r) for r in rows]
        return tuple(np.stack(x) for x in zip(*parts))
    if p.base == "NVQ1-S":
        return np.stack([np.stack([nvq1._unpack_table(r[:1024], 512), nvq1._unpack_table(r[1024:], 512)]) for r in rows])
    return np.stack([nvq1._unpack_table(r, 2048) for r in rows])


def pack_bank(p: NepqProfile, *tables) -> np.ndarray:
    """One bank of the pool from decoded tables: NPQ0 bases ``(ladder, first, second)``; NVQ1-S ``([2, 512, 8],)``;
    NVQ1-L ``([2048, 8],)``."""
    p = profile_of(p)
    if p.base.startswith("NPQ0"):
        raw = npq0.pack_tables(npq0.VARIANTS[p.base], *tables)
    elif p.base == "NVQ1-S":
        t = np.asarray(tables[0])
        raw = nvq1._pack_table(t[0], 512) + nvq1._pack_table(t[1], 512)
    else:
        raw = nvq1._pack_table(np.asarray(tables[0]), 2048)
    if len(raw) != p.bank_bytes:
        raise ValueError(f"{p.label}: a bank is {p.bank_bytes} bytes, got {len(raw)}")
    return np.frombuffer(raw, dtype=np.uint8).copy()


def _check(t: NepqTensor):
    p = profile_of(t.profile)
    shape = tuple(int(s) for s in t.shape)
    if len(shape) != 3 or min(shape) <= 0 or shape[2] % VEC:
        raise ValueError(f"{p.label}: the shape must be (experts, out, K) with K a positive multiple of 8, got {shape}")
    e, o, k = shape
    ng, nv, ns = p.geometry(k)
    banks = np.asarray(t.banks)
    if banks.ndim != 2 or banks.shape[1] != p.bank_bytes or not 1 <= banks.shape[0] <= 256:
        raise ValueError(f"{p.label}: the pool must be [1..256, {p.bank_bytes}] bytes, got {banks.shape}")
    _decode_banks(p, banks)  # every bank must be a valid table set of the base format
    want = {"anchors": (e, o), "state": (e, o, ng), "indices": (e, o, nv), "bank_ids": (e, o, ns)}
    for name, shp in want.items():
        if np.asarray(getattr(t, name)).shape != shp:
            raise ValueError(f"{p.label}: {name} must have shape {shp}, got {np.asarray(getattr(t, name)).shape}")
    with np.errstate(over="ignore", invalid="ignore"):
        a16 = np.asarray(t.anchors, dtype=np.float32).astype(np.float16)
    if not np.isfinite(a16).all() or (a16 < 0).any():
        raise ValueError(f"{p.label}: anchors must be finite and non-negative in FP16")
    for name, bits in (("state", p.state_bits), ("indices", p.index_bits)):
        a = np.asarray(getattr(t, name))
        if not np.issubdtype(a.dtype, np.integer) or (a.size and (a.min() < 0 or int(a.max()) >> bits)):
            raise ValueError(f"{p.label}: {name} must be integers below 2**{bits}")
    ids = np.asarray(t.bank_ids)
    if not np.issubdtype(ids.dtype, np.integer) or ids.min() < 0 or ids.max() >= banks.shape[0]:
        raise ValueError(f"{p.label}: a bank id points outside the pool")
    if p.aux_bits:
        aux = np.asarray(t.aux) if t.aux is not None else None
        if aux is None or aux.shape != (e, o, ng) or not np.issubdtype(aux.dtype, np.integer) or aux.min() < 0 or aux.max() > 1:
            raise ValueError(f"{p.label}: aux must be a 0/1 array of shape {(e, o, ng)}")
    elif t.aux is not None and np.asarray(t.aux).size:
        raise ValueError(f"{p.label} has no aux stream")
    block, seed = int(t.rotation_block), int(t.rotation_seed)
    if block:
        if block & (block - 1) or k % block or not 0 <= seed < 1 << 64:
            raise ValueError(f"{p.label}: the rotation block must be a power of two dividing K, the seed a uint64")
    elif seed:
        raise ValueError(f"{p.label}: a rotation seed needs a rotation block")
    r = t.residual
    if not p.residual_block:
        if r is not None:
            raise ValueError(f"{p.label} carries no residual")
        return ng, nv, ns
    if r is None or not block:
        raise ValueError(f"{p.label} needs a residual section and a rotation")
    if not 0 <= int(r.padding) < 1 << 32:
        raise ValueError(f"{p.label}: residual padding must fit 32 bits")
    with np.errstate(over="ignore", invalid="ignore"):
        d16 = np.asarray(r.dictionary, dtype=np.float32).astype(np.float16)
    if d16.shape != (DICTIONARY, VEC) or not np.isfinite(d16).all():
        raise ValueError(f"{p.label}: the residual dictionary must be a finite [{DICTIONARY}, {VEC}] FP16 array")
    bpr = t.blocks_per_row
    first = np.asarray(r.first)
    if first.shape != (e, o, bpr):
        raise ValueError(f"{p.label}: first residual records must have shape {(e, o, bpr)}")
    _check_records(p, first.reshape(-1), np.arange(first.size), nv, bpr, "first")
    if p.residual_second:
        mask = np.asarray(r.second_mask) if r.second_mask is not None else None
        if mask is None or mask.shape != (e, o, bpr) or np.any((mask != 0) & (mask != 1)):
            raise ValueError(f"{p.label}: the second-record mask must be a 0/1 array of shape {(e, o, bpr)}")
        rec = np.asarray(r.second_records if r.second_records is not None else np.empty(0, np.uint16))
        where = np.flatnonzero(mask.reshape(-1))
        if rec.ndim != 1 or rec.size != where.size:
            raise ValueError(f"{p.label}: {rec.size} second records for {where.size} marked blocks")
        _check_records(p, rec, where, nv, bpr, "second")
    elif r.second_mask is not None or r.second_records is not None:
        raise ValueError(f"{p.label} has no second residual stream")
    return ng, nv, ns


def _check_records(p: NepqProfile, records, block_ids, nv: int, bpr: int, name: str) -> None:
    rec = np.asarray(records)
    if not np.issubdtype(rec.dtype, np.integer):
        raise ValueError(f"{p.label}: {name} residual records must be integers")
    rec = rec.astype(np.int64)
    if rec.size == 0:
        return
    if rec.min() < 0 or int(rec.max()) >> p.record_bits:
        raise ValueError(f"{p.label}: a {name} residual record exceeds {p.record_bits} bits")
    pos = rec & ((1 << p.position_bits) - 1)
    room = np.minimum(p.residual_block, nv - (np.asarray(block_ids) % bpr) * p.residual_block)
    if (pos >= room).any():
        raise ValueError(f"{p.label}: a {name} residual position lies outside its block")


def pack_nepq(t: NepqTensor) -> bytes:
    _check(t)
    p = profile_of(t.profile)
    e, o, k = (int(s) for s in t.shape)
    banks = np.ascontiguousarray(t.banks, dtype=np.uint8)
    parts = [
        _HEAD.pack(b"NEP1", 1, p.profile_id, SUPER, 1 if t.rotation_block else 0, e, o, k, banks.shape[0],
                   int(t.rotation_block), int(t.rotation_seed)),
        banks.tobytes(),
        np.asarray(t.anchors, dtype=np.float32).astype("<f2").tobytes(),
        pack_bits(np.asarray(t.state).reshape(-1), p.state_bits),
        pack_bits(np.asarray(t.indices).reshape(-1), p.index_bits),
        pack_bits(np.asarray(t.aux).reshape(-1), 1) if p.aux_bits else b"",
        np.ascontiguousarray(t.bank_ids, dtype=np.uint8).tobytes(),
    ]
    if p.residual_block:
        r = t.residual
        second = np.asarray(r.second_records if r.second_records is not None else np.empty(0, np.uint16))
        parts += [
            _RES_HEAD.pack(b"NRA1", 1, p.record_bits, p.position_bits, 1 if p.residual_second else 0, DICTIONARY,
                           t.rows * t.blocks_per_row, int(second.size), int(r.padding), 0),
            np.asarray(r.dictionary, dtype=np.float32).astype("<f2").tobytes(),
            pack_bits(np.asarray(r.first).reshape(-1), p.record_bits),
        ]
        if p.residual_second:
            parts += [pack_bits(np.asarray(r.second_mask).reshape(-1), 1), pack_bits(second, p.record_bits) if second.size else b""]
        parts.append(bytes(int(r.padding)))
    return b"".join(parts)


def unpack_nepq(blob) -> NepqTensor:
    blob = memoryview(blob)
    if len(blob) < _HEAD.size:
        raise ValueError("truncated NEPQ header")
    magic, version, pid, per_super, flags, e, o, k, nbanks, block, seed = _HEAD.unpack_from(blob)
    if bytes(magic) != b"NEP1" or version != 1:
        raise ValueError("not a NEPQ blob of a known version")
    p = profile_of(pid)
    if per_super != SUPER or flags & ~1 or bool(flags & 1) != bool(block):
        raise ValueError(f"{p.label}: unsupported super-group size or inconsistent rotation flag")
    if min(e, o, k) <= 0 or k % VEC or not 1 <= nbanks <= 256:
        raise ValueError(f"{p.label}: invalid dimensions")
    rows = e * o
    ng, nv, ns = p.geometry(k)
    off = _HEAD.size
    if off + nbanks * p.bank_bytes + 2 * rows > len(blob):
        raise ValueError(f"{p.label}: truncated pool or anchors")
    banks = np.frombuffer(blob, dtype=np.uint8, count=nbanks * p.bank_bytes, offset=off).reshape(nbanks, p.bank_bytes).copy()
    off += nbanks * p.bank_bytes
    anchors = np.frombuffer(blob, dtype="<f2", count=rows, offset=off).astype(np.float32).reshape(e, o)
    off += 2 * rows
    state, off = unpack_bits(blob, off, rows * ng, p.state_bits)
    idx, off = unpack_bits(blob, off, rows * nv, p.index_bits)
    aux = None
    if p.aux_bits:
        aux, off = unpack_bits(blob, off, rows * ng, 1)
        aux = aux.astype(np.uint8).reshape(e, o, ng)
    if off + rows * ns > len(blob):
        raise ValueError(f"{p.label}: truncated bank ids")
    bank_ids = np.frombuffer(blob, dtype=np.uint8, count=rows * ns, offset=off).reshape(e, o, ns).copy()
    off += rows * ns
    residual = None
    if p.residual_block:
        if off + _RES_HEAD.size > len(blob):
            raise ValueError(f"{p.label}: truncated residual header")
        rmagic, rver, rbits, pbits, rflags, entries, blocks, nsecond, padding, reserved = _RES_HEAD.unpack_from(blob, off)
        bpr = math.ceil(nv / p.residual_block)
        if (bytes(rmagic) != b"NRA1" or rver != 1 or rbits != p.record_bits or pbits != p.position_bits or entries != DICTIONARY
                or rflags != (1 if p.residual_second else 0) or blocks != rows * bpr or reserved
                or any(blob[off + _RES_HEAD.size - 32 : off + _RES_HEAD.size]) or (nsecond and not p.residual_second)):
            raise ValueError(f"{p.label}: unsupported residual section")
        off += _RES_HEAD.size
        if off + DICTIONARY * VEC * 2 > len(blob):
            raise ValueError(f"{p.label}: truncated residual dictionary")
        dictionary = np.frombuffer(blob, dtype="<f2", count=DICTIONARY * VEC, offset=off).astype(np.float32).reshape(DICTIONARY, VEC)
        off += DICTIONARY * VEC * 2
        first, off = unpack_bits(blob, off, blocks, p.record_bits)
        mask = second = None
        if p.residual_second:
            mask, off = unpack_bits(blob, off, blocks, 1)
            if int(mask.sum()) != nsecond:
                raise ValueError(f"{p.label}: the second-record count does not match its mask")
            second = np.empty(0, np.uint16)
            if nsecond:
                second, off = unpack_bits(blob, off, nsecond, p.record_bits)
            mask = mask.astype(np.uint8).reshape(e, o, bpr)
        if off + padding > len(blob) or any(blob[off : off + padding]):
            raise ValueError(f"{p.label}: residual padding is truncated or not zero")
        off += padding
        residual = NepqResidual(dictionary, first.astype(np.uint16).reshape(e, o, bpr), mask,
                                None if second is None else second.astype(np.uint16), int(padding))
    if off != len(blob):
        raise ValueError(f"{p.label}: {len(blob) - off} stray bytes at the end")
    t = NepqTensor(p, (e, o, k), anchors, state.astype(np.uint8).reshape(e, o, ng),
                   idx.astype(np.uint16 if p.index_bits > 8 else np.uint8).reshape(e, o, nv), aux, bank_ids, banks,
                   int(block), int(seed), residual)
    _check(t)
    return t


def dequantize_nepq_rows(t: NepqTensor, start: int, stop: int, *, decoded=None) -> np.ndarray:
    """Flattened rows ``[start, stop)`` (row = expert * out + neuron) in STORED coordinates, float32 ``[n, K]``."""
    p = profile_of(t.profile)
    k = int(t.shape[2])
    ng, nv, _ns = p.geometry(k)
    rows = t.rows
    if not 0 <= start <= stop <= rows:
        raise ValueError(f"row range [{start}, {stop}) outside {rows} rows")
    n = stop - start
    state = np.asarray(t.state, dtype=np.uint8).reshape(rows, ng)[start:stop]
    idx = np.asarray(t.indices).reshape(rows, nv)[start:stop].astype(np.int64)
    anchors = np.asarray(t.anchors, dtype=np.float32).reshape(rows)[start:stop]
    gbank = np.repeat(np.asarray(t.bank_ids, dtype=np.uint8).reshape(rows, -1)[start:stop], SUPER, axis=1)[:, :ng].astype(np.int64)
    vbank = np.repeat(gbank, GROUP // VEC, axis=1)[:, :nv]
    vstate = np.repeat(state, GROUP // VEC, axis=1)[:, :nv].astype(np.int64)
    tables = _decode_banks(p, t.banks) if decoded is None else decoded
    if p.base.startswith("NPQ0"):
        ladder, first, second = tables
        v = npq0.VARIANTS[p.base]
        code = np.concatenate([first[vbank, vstate, idx & ((1 << v.first_bits) - 1)], second[vbank, vstate, idx >> v.first_bits]], -1)
        scale = anchors[:, None] * ladder[gbank, state.astype(np.int64)]
        out = code.reshape(n, k).astype(np.float32) * np.repeat(scale, GROUP, axis=1)[:, :k]
    else:
        aux = np.asarray(t.aux, dtype=np.uint8).reshape(rows, ng)[start:stop]
        delta = np.float32(_NVQ1_BASE[p.base].delta)
        if p.base == "NVQ1-S":
            code = tables[vbank, np.repeat(aux, GROUP // VEC, axis=1)[:, :nv].astype(np.int64), idx]
        else:
            code = tables[vbank, idx]
        shift = np.where(aux != 0, -delta, delta).astype(np.float32)
        scale = anchors[:, None] * state.astype(np.float32)
        out = np.repeat(scale, GROUP, axis=1)[:, :k] * (code.reshape(n, k).astype(np.float32) + np.repeat(shift, GROUP, axis=1)[:, :k])
    if p.residual_block and n:
        _add_residual(t, out, start, stop)
    return out


def _residual_entries(t: NepqTensor, start: int, stop: int):
    """(row - start, vector, dictionary id) of every residual record in the row range."""
    p, r, bpr = t.profile, t.residual, t.blocks_per_row
    pmask = (1 << p.position_bits) - 1
    first = np.asarray(r.first).reshape(-1, bpr)[start:stop].astype(np.int64)
    rr, bb = np.meshgrid(np.arange(stop - start), np.arange(bpr), indexing="ij")
    parts = [(rr.reshape(-1), (bb * p.residual_block + (first & pmask)).reshape(-1), (first >> p.position_bits).reshape(-1))]
    if p.residual_second:
        mask = np.asarray(r.second_mask, dtype=np.uint8).reshape(-1)
        dense = np.full(mask.size, -1, dtype=np.int64)
        dense[np.flatnonzero(mask)] = np.asarray(r.second_records, dtype=np.int64)
        sec = dense.reshape(-1, bpr)[start:stop]
        on = sec >= 0
        parts.append((rr[on], bb[on] * p.residual_block + (sec[on] & pmask), sec[on] >> p.position_bits))
    return parts


def _add_residual(t: NepqTensor, out: np.ndarray, start: int, stop: int) -> None:
    dictionary = np.asarray(t.residual.dictionary, dtype=np.float32)
    view = out.reshape(out.shape[0], -1, VEC)
    for rows, vecs, ids in _residual_entries(t, start, stop):
        np.add.at(view, (rows, vecs), dictionary[ids])


def dequantize_nepq(t: NepqTensor, *, logical: bool = True) -> np.ndarray:
    """``[experts, out, K]`` float32.  ``logical=False`` returns the stored (rotated) coordinates, the form a runtime
    that rotates its activations multiplies with."""
    _check(t)
    out = dequantize_nepq_rows(t, 0, t.rows).reshape(t.shape)
    if logical and t.rotation_block:
        out = unrotate_rows(out, t.rotation_block, t.rotation_seed)
    return out.astype(np.float32)


def residual_by_vector(t: NepqTensor):
    """The residual records regrouped by input vector, for products that walk the K axis: CSR ``offsets [vectors + 1]``,
    then per record its flattened row and dictionary id (``mfq/formats/nepq.py:923-984`` builds the same index)."""
    nv = t.shape[2] // VEC
    parts = _residual_entries(t, 0, t.rows)
    rows = np.concatenate([p[0] for p in parts])
    vecs = np.concatenate([p[1] for p in parts])
    ids = np.concatenate([p[2] for p in parts])
    order = np.argsort(vecs, kind="stable")
    offsets = np.zeros(nv + 1, dtype=np.uint32)
    np.cumsum(np.bincount(vecs, minlength=nv), out=offsets[1:])
    return offsets, rows[order].astype(np.uint32), ids[order].astype(np.uint16)


# ---- encoder -------------------------------------------------------------------------------------------------------------
def _score_npq0(x, anchors, tables, v: npq0.Npq0Variant, live):
    """Best (state, index) of every group under ONE bank for fixed anchors.  ``x [R, G, 3, 8]`` torch; ``live [G, 3]``
    is false for the padding vectors of a short last group, which cost nothing.  Returns (error [R, G], state [R, G],
    index [R, G, 3])."""
    import torch
    ladder, first, second = (torch.as_tensor(np.asarray(a, dtype=np.float32), device=x.device) for a in tables)
    r, g = x.shape[:2]
    halves = (x[..., :4], x[..., 4:])
    best = torch.full((r, g), float("inf"), device=x.device)
    best_s = torch.zeros((r, g), dtype=torch.int64, device=x.device)
    best_i = torch.zeros((r, g, 3), dtype=torch.int64, device=x.device)
    for s in range(v.states):
        scale = (anchors * ladder[s])[:, None, None, None, None]                    # [R, 1, 1, 1, 1]
        err = torch.zeros((r, g), device=x.device)
        idx = torch.zeros((r, g, 3), dtype=torch.int64, device=x.device)
        for h, (xs, book) in enumerate(zip(halves, (first[s], second[s]))):
            cand = scale * book[None, None, None]                                   # [R, 1, 1, n, 4]
            d = ((xs[:, :, :, None, :] - cand) ** 2).sum(-1)                        # [R, G, 3, n]
            val, arg = d.min(-1)
            err = err + (val * live[None]).sum(-1)
            idx = idx | (arg << (0 if h == 0 else v.first_bits))
        better = err < best
        best = torch.where(better, err, best)
        best_s = torch.where(better, torch.full_like(best_s, s), best_s)
        best_i = torch.where(better[..., None], idx, best_i)
    return best, best_s, best_i


def _basis_npq0(state, idx, gbank, pool, v: npq0.Npq0Variant):
    """ladder * code per weight for a mixed-bank assignment: [R, G, 3, 8]."""
    import torch
    ladder, first, second = pool
    vb = gbank[..., None].expand(-1, -1, 3)
    vs = state[..., None].expand(-1, -1, 3)
    code = torch.cat([first[vb, vs, idx & ((1 << v.first_bits) - 1)], second[vb, vs, idx >> v.first_bits]], -1)
    return code * ladder[gbank, state][..., None, None]


def _kmeans(points, k: int, iterations: int, seed: int):
    """Plain Lloyd on torch ``points [n, d]``; returns ``[k, d]`` (unused centres stay at their seeds; zeros if n == 0)."""
    import torch
    n = points.shape[0]
    if n == 0:
        return torch.zeros((k, points.shape[1]), device=points.device)
    g = torch.Generator().manual_seed(seed)
    pick = torch.randperm(n, generator=g)[:k] if n >= k else torch.randint(0, n, (k,), generator=g)
    cent = points[pick.to(points.device)].clone()
    if n < k:
        cent[n:] = 0
    for _ in range(iterations):
        a = torch.cdist(points, cent).argmin(1)
        sums = torch.zeros_like(cent).index_add_(0, a, points)
        cnt = torch.zeros(k, device=points.device).index_add_(0, a, torch.ones(n, device=points.device))
        cent = torch.where(cnt[:, None] > 0, sums / cnt.clamp_min(1)[:, None], cent)
    return cent


def train_pool(stored: np.ndarray, profile, banks: int, *, seed: int = 0, device: str | None = None) -> np.ndarray:
    """A pool of ``banks`` table sets for ``stored [experts, out, K]``: bank ``b`` is what the base format's own table
    fitting finds on the ``b``-th contiguous slice of the experts (the ternary L base keeps the IQ1_S grid as bank 0)."""
    p = profile_of(profile)
    e = stored.shape[0]
    banks = max(1, min(int(banks), 256))
    out = []
    for b in range(banks):
        lo, hi = (b * e) // banks, max((b * e) // banks + 1, ((b + 1) * e) // banks)
        part = stored[lo:min(hi, e)].reshape(-1, stored.shape[2]) if lo < e else stored.reshape(-1, stored.shape[2])
        if p.base.startswith("NPQ0"):
            q = npq0.quantize_npq0(part, npq0.VARIANTS[p.base], seed=seed + b)
            out.append(pack_bank(p, q.scale_lut, q.first_codebooks, q.second_codebooks))
        elif p.base == "NVQ1-S":
            q = nvq1.quantize_nvq1(part, "NVQ1-S", device=device)
            out.append(pack_bank(p, q.table))
        else:
            table = nvq1.IQ1S_GRID
            if b:
                q = nvq1.quantize_nvq1(part, "NVQ1-L", train_table=True, device=device)
                table = nvq1.IQ1S_GRID if q.table is None else q.table
            out.append(pack_bank(p, table))
    return np.stack(out)


def quantize_nepq(weight, profile="NEPQ0-S", *, banks: int = 4, pool: np.ndarray | None = None, rotation_block: int | None = None,
                  rotation_seed: int = 0, iterations: int = 2, second_fraction: float = 0.5, seed: int = 0,
                  device: str | None = None, row_chunk: int = 256) -> NepqTensor:
    """Encode ``weight [experts, out, K]`` (K a multiple of 8).  ``pool``: a frozen ``[banks, bank bytes]`` pool (as
    :func:`train_pool` or another tensor's ``banks``); by default one is trained on this tensor.  ``rotation_block``:
    0 none, None = none for the plain profiles and the largest power of two <= 128 dividing K for the ``-A`` profiles
    (which require one).  ``second_fraction``: share of blocks that get a second residual record (NEPQ1-A)."""
    import torch
    p = profile_of(profile)
    w = np.asarray(weight, dtype=np.float32)
    if w.ndim != 3 or w.shape[2] % VEC:
        raise ValueError(f"{p.label}: expected [experts, out, K] with K a multiple of 8, got {w.shape}")
    e, o, k = w.shape
    if rotation_block is None:
        rotation_block = 0
        if p.residual_block:
            rotation_block = 128
            while k % rotation_block:
                rotation_block //= 2
    if p.residual_block and not rotation_block:
        raise ValueError(f"{p.label} needs a rotation block")
    if not rotation_block:
        rotation_seed = 0
    stored = rotate_rows(w.reshape(-1, k), rotation_block, rotation_seed).reshape(w.shape) if rotation_block else w
    pool_bytes = train_pool(stored, p, banks, seed=seed, device=device) if pool is None else np.ascontiguousarray(pool, dtype=np.uint8)
    nb = pool_bytes.shape[0]
    decoded = _decode_banks(p, pool_bytes)
    dev = torch.device(device or "cpu")
    ng, nv, ns = p.geometry(k)
    rows = e * o
    flat = stored.reshape(rows, k)
    anchors_o = np.zeros(rows, dtype=np.float32)
    state_o = np.zeros((rows, ng), dtype=np.uint8)
    idx_o = np.zeros((rows, nv), dtype=np.uint16 if p.index_bits > 8 else np.uint8)
    aux_o = np.zeros((rows, ng), dtype=np.uint8) if p.aux_bits else None
    bank_o = np.zeros((rows, ns), dtype=np.uint8)
    is_pq = p.base.startswith("NPQ0")
    if is_pq:
        v = npq0.VARIANTS[p.base]
        pool_t = tuple(torch.as_tensor(np.asarray(a, dtype=np.float32), device=dev) for a in decoded)
        top = float(max(np.abs(decoded[1]).max(), np.abs(decoded[2]).max()) * decoded[0].max())
    else:
        v = _NVQ1_BASE[p.base]
        tabs = torch.as_tensor(np.asarray(decoded, dtype=np.float32), device=dev)
        pool_t = tabs if p.base == "NVQ1-S" else torch.stack([tabs, tabs], 1)    # [B, 2, entries, 8]
        top = float(((1 << v.sub_bits) - 1) * (1.0 + v.delta))
    super_of_group = torch.arange(ng, device=dev) // SUPER
    live = (torch.arange(ng * 3, device=dev) < nv).reshape(ng, 3).float()
    for r0 in range(0, rows, row_chunk):
        r1 = min(rows, r0 + row_chunk)
        n = r1 - r0
        x = torch.zeros((n, ng * GROUP), dtype=torch.float32, device=dev)
        x[:, :k] = torch.from_numpy(flat[r0:r1]).to(dev)
        xg = x.reshape(n, ng, 3, VEC)
        anchors = (x.abs().amax(1) / top).clamp_min(1e-8).half().float()
        state = idx = aux = gbank = None
        for _ in range(max(1, iterations) + 1):
            errs, cands = [], []
            for b in range(nb):
                if is_pq:
                    err, st, ix = _score_npq0(xg, anchors, tuple(a[b] for a in decoded), v, live)
                    ax = None
                else:
                    xv = x[:, : nv * VEC].reshape(n, nv, VEC)
                    st, ax, ix = nvq1._assign(xv, torch.ones_like(xv), anchors, pool_t[b], v, row_chunk)
                    basis = nvq1._basis(st, ax, ix, pool_t[b], v, nv)
                    e_vec = ((xv - anchors[:, None, None] * basis) ** 2).sum(-1)
                    e_vec = torch.cat([e_vec, e_vec.new_zeros(n, ng * 3 - nv)], 1)
                    err = e_vec.reshape(n, ng, 3).sum(-1)
                    ix = torch.cat([ix, ix.new_zeros(n, ng * 3 - nv)], 1).reshape(n, ng, 3)
                errs.append(torch.zeros((n, ns), device=dev).index_add_(1, super_of_group, err))
                cands.append((st, ax, ix))
            pick = torch.stack(errs).argmin(0)                                       # [n, super-groups]
            gbank = pick[:, super_of_group]                                          # [n, groups]
            state = torch.stack([c[0] for c in cands]).gather(0, gbank[None])[0]
            idx = torch.stack([c[2] for c in cands]).gather(0, gbank[None, :, :, None].expand(1, n, ng, 3))[0]
            if not is_pq:
                aux = torch.stack([c[1] for c in cands]).gather(0, gbank[None])[0]
            # least-squares anchors for this assignment
            if is_pq:
                basis = _basis_npq0(state, idx, gbank, pool_t, v)
            else:
                vb = gbank[..., None].expand(-1, -1, 3)
                va = aux[..., None].expand(-1, -1, 3)
                code = pool_t[vb, va, idx] + torch.where(va != 0, -v.delta, v.delta)[..., None]
                basis = code * state[..., None, None].float()
            basis = basis * live[None, :, :, None]
            num, den = (xg * basis).sum((1, 2, 3)), (basis * basis).sum((1, 2, 3))
            anchors = torch.where(den > 0, num / den.clamp_min(1e-30), anchors).clamp(0, 65504.0).half().float()
        anchors_o[r0:r1] = anchors.cpu().numpy()
        state_o[r0:r1] = state.cpu().numpy().astype(np.uint8)
        idx_o[r0:r1] = idx.reshape(n, ng * 3)[:, :nv].cpu().numpy().astype(idx_o.dtype)
        bank_o[r0:r1] = gbank[:, ::SUPER].cpu().numpy().astype(np.uint8)
        if aux_o is not None:
            aux_o[r0:r1] = aux.cpu().numpy().astype(np.uint8)
    t = NepqTensor(p, (e, o, k), anchors_o.reshape(e, o), state_o.reshape(e, o, ng), idx_o.reshape(e, o, nv),
                   None if aux_o is None else aux_o.reshape(e, o, ng), bank_o.reshape(e, o, ns), pool_bytes,
                   int(rotation_block), int(rotation_seed))
    if p.residual_block:
        t.residual = _fit_residual(t, flat, second_fraction, seed, dev)
    _check(t)
    return t


def _fit_residual(t: NepqTensor, stored: np.ndarray, second_fraction: float, seed: int, dev) -> NepqResidual:
    """Dictionary = k-means over the worst vector of every block; a record = the (position, entry) that removes the most
    error in its block; NEPQ1-A: the ``second_fraction`` of blocks where a second record removes the most get one."""
    import torch
    p = t.profile
    rows, k = stored.shape
    nv, bpr, bv = k // VEC, t.blocks_per_row, p.residual_block
    plain = NepqTensor(**{**t.__dict__, "profile": profile_of(p.base.replace("NPQ0", "NEPQ0").replace("NVQ1", "NEPQ1")), "residual": None})
    base = dequantize_nepq_rows(plain, 0, rows)
    res = torch.from_numpy(stored - base).to(dev).reshape(rows, nv, VEC)
    pad = bpr * bv - nv
    if pad:
        res = torch.cat([res, res.new_zeros(rows, pad, VEC)], 1)
    live = (torch.arange(bpr * bv, device=dev) < nv).reshape(bpr, bv)
    blocks = res.reshape(rows, bpr, bv, VEC)
    worst = blocks.pow(2).sum(-1).argmax(-1)                                           # [rows, bpr]
    train = blocks.gather(2, worst[..., None, None].expand(-1, -1, 1, VEC)).reshape(-1, VEC)
    if train.shape[0] > 200_000:
        g = torch.Generator().manual_seed(seed)
        train = train[torch.randperm(train.shape[0], generator=g)[:200_000].to(dev)]
    dictionary = _kmeans(train, DICTIONARY, 8, seed)
    dictionary[dictionary.pow(2).sum(-1).argmin()] = 0.0   # a block nothing helps can then add nothing
    dictionary = dictionary.half().float()

    def best_records(blk):
        """Per block: the (position, entry) with the largest error reduction |r|^2 - |r - d|^2, and that reduction."""
        flatv = blk.reshape(-1, VEC)
        gain = torch.empty(flatv.shape[0], device=dev)
        ident = torch.empty(flatv.shape[0], dtype=torch.int64, device=dev)
        dn = dictionary.pow(2).sum(-1)
        for s in range(0, flatv.shape[0], 65536):
            sc = 2.0 * flatv[s : s + 65536] @ dictionary.T - dn[None]
            gain[s : s + 65536], ident[s : s + 65536] = sc.max(1)
        gain = gain.reshape(rows, bpr, bv).masked_fill(~live[None], float("-inf"))
        ident = ident.reshape(rows, bpr, bv)
        g, pos = gain.max(-1)
        return g, pos, ident.gather(2, pos[..., None])[..., 0]

    _g, pos, ident = best_records(blocks)
    first = (ident << p.position_bits | pos).cpu().numpy().astype(np.uint16)
    mask = second = None
    if p.residual_second:
        picked = dictionary[ident]                                                     # [rows, bpr, 8]
        blocks = blocks.clone()
        blocks.scatter_add_(2, pos[..., None, None].expand(-1, -1, 1, VEC), -picked[:, :, None, :])
        g2, pos2, id2 = best_records(blocks)
        count = int(round(max(0.0, min(1.0, second_fraction)) * g2.numel()))
        flat_gain = g2.reshape(-1)
        chosen = torch.zeros_like(flat_gain, dtype=torch.bool)
        if count:
            top = flat_gain.topk(count).indices
            chosen[top] = flat_gain[top] > 0
        mask = chosen.reshape(rows, bpr).cpu().numpy().astype(np.uint8)
        second = (id2 << p.position_bits | pos2).reshape(-1)[chosen].cpu().numpy().astype(np.uint16)
    e, o, _ = t.shape
    return NepqResidual(dictionary.cpu().numpy(), first.reshape(e, o, bpr), None if mask is None else mask.reshape(e, o, bpr), second)
