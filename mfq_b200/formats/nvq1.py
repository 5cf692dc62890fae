"""NVQ1-L / NVQ1-S: neuron-anchored ternary vector quantization at 1.3 - 1.7 bits per weight.

A weight row (one output neuron) is cut into groups of 24 weights = three 8-vectors.  Every 8-vector is an entry of a
ternary codebook ({-1, 0, 1}^8); a group shares one integer sub-scale ``q`` and one sign bit that shifts all its entries
by ``+delta`` or ``-delta``; a row shares one FP16 anchor ``a``:

    w[8 v .. 8 v + 7]  ~=  a * q[group] * (codebook[index[v]] + (-1)^sign[group] * delta)

* **NVQ1-L**: the 2048-entry ternary grid of llama.cpp's IQ1_S (11-bit indices), ``delta`` = 1/8, 3- or 4-bit sub-scales,
  group size any multiple of 8 (24 by default) -- 1.54 / 1.58 bits per weight plus 16 bits per row.  A tensor may carry
  its own 2048-entry table instead (profile 2).
* **NVQ1-S**: two 512-entry tables ("banks", 9-bit indices) carried IN every blob, the sign bit also selects the bank,
  ``delta`` = 5/32, 4-bit sub-scales: exactly 32 bits per complete group = 1.33 bits per weight plus 16 per row.

Byte layout (little endian, bit streams LSB first, each stream runs across the whole tensor):

    "NQ1L" | profile u8 (1 grid, 2 own table) | sub_bits u8 | groupsize u16 | axis i32 | row length i32 | ndim u32
    "NQ1S" | version u8 (1)                   | sub_bits u8 | groupsize u16 | axis i32 | row length i32 | ndim u32
    shape ndim x i64 | rows u32 | [table: 4096 B (L, profile 2) / 2 x 1024 B (S)] | anchors rows x f16
    | sub-scales | indices | sign bits

A table entry is packed as 8 base-4 digits (value + 1) in a little-endian u16.

The encoder here is a batched search in torch (CPU or GPU): for a fixed anchor every group tries both signs and every
sub-scale, each 8-vector taking its best entry (one ``[vectors, 8] x [8, entries]`` product per sign), then the anchor is
refitted by least squares; NVQ1-S additionally re-estimates its two tables from the assigned vectors (Lloyd steps on the
ternary alphabet).  Optional per-column importance weights enter every error term.

Reference: ``mfq/formats/nvq1_l.py`` (layout :232-351, grid :21-111), ``mfq/formats/nvq1_s.py`` (:150-351),
``mfq/quantize/nvq1_l_quant.py`` (``_assign_groups`` :56, ``dequantize`` :384).  The grid is the public IQ1_S table of
llama.cpp (MIT licence), shipped as ``data/iq1s_grid.bin`` and checked against its SHA-256.
"""

from __future__ import annotations

import hashlib
import math
import struct
from dataclasses import dataclass
from pathlib import Path

import numpy as np

_GRID_SHA256 = "e9ffebfc997ad6023063a667c0bf4eedd8ebf7f56b3da399cbc7d1b1f7ea52c6"
_HEADER = struct.Struct("<4sBBHiiI")


def _unpack_table(raw: bytes, entries: int) -> np.ndarray:
    if len(raw) != 2 * entries:
        raise ValueError(f"a packed ternary table of {entries} entries is {2 * entries} bytes, got {len(raw)}")
    enc = np.frombuffer(raw, dtype="<u2")
    digits = (enc[:, None] >> (2 * np.arange(8, dtype=np.uint16))[None, :]) & 3
    if (digits > 2).any():
        raise ValueError("packed ternary table holds a digit outside {0, 1, 2}")
    return np.ascontiguousarray(digits.astype(np.int8) - 1)


def _pack_table(table: np.ndarray, entries: int) -> bytes:
    t = np.asarray(table)
    if t.shape != (entries, 8) or not np.isin(t, (-1, 0, 1)).all():
        raise ValueError(f"a ternary table must be [{entries}, 8] over {{-1, 0, 1}}")
    if np.unique(t, axis=0).shape[0] != entries:
        raise ValueError("ternary table entries must be unique")
    digits = (t.astype(np.int16) + 1).astype(np.uint16)
    return np.bitwise_or.reduce(digits << (2 * np.arange(8, dtype=np.uint16))[None, :], axis=1).astype("<u2").tobytes()


def _load_grid() -> np.ndarray:
    raw = (Path(__file__).parent / "data" / "iq1s_grid.bin").read_bytes()
    if hashlib.sha256(raw).hexdigest() != _GRID_SHA256:
        raise RuntimeError("data/iq1s_grid.bin does not match its checksum")
    grid = _unpack_table(raw, 2048)
    grid.setflags(write=False)
    return grid


IQ1S_GRID = _load_grid()


@dataclass(frozen=True)
class Nvq1Variant:
    label: str          # container dtype string
    magic: bytes
    index_bits: int
    delta: float
    banked: bool        # two tables selected by the sign bit, always stored in the blob
    sub_bits: int
    groupsize: int = 24

    @property
    def entries(self) -> int:
        return 1 << self.index_bits

    def default_table(self) -> np.ndarray:
        """The grid (L); for S a starting point for training: every fourth grid entry in both banks."""
        if not self.banked:
            return IQ1S_GRID
        return np.stack([IQ1S_GRID[::4], IQ1S_GRID[::4]])

    def stream_nbytes(self, rows: int, row_len: int) -> int:
        ng, nv = math.ceil(row_len / self.groupsize), math.ceil(row_len / 8)
        return 2 * rows + (rows * ng * self.sub_bits + 7) // 8 + (rows * nv * self.index_bits + 7) // 8 + (rows * ng + 7) // 8

    def bits_per_weight(self, rows: int, row_len: int, include_table: bool = True) -> float:
        table = 2 * 2 * self.entries if (self.banked and include_table) else 0
        return 8.0 * (table + self.stream_nbytes(rows, row_len)) / (rows * row_len)


NVQ1_L_S3 = Nvq1Variant("NVQ1-L", b"NQ1L", 11, 0.125, False, 3)
NVQ1_L_S4 = Nvq1Variant("NVQ1-L", b"NQ1L", 11, 0.125, False, 4)
NVQ1_S = Nvq1Variant("NVQ1-S", b"NQ1S", 9, 0.15625, True, 4)
VARIANTS = {"NVQ1-L": NVQ1_L_S3, "NVQ1-L-S3": NVQ1_L_S3, "NVQ1-L-S4": NVQ1_L_S4, "NVQ1-S": NVQ1_S}
DTYPES = ("NVQ1-L", "NVQ1-S")


@dataclass
class Nvq1Tensor:
    variant: Nvq1Variant
    shape: tuple[int, ...]
    axis: int                 # the axis that indexes rows (output neurons)
    row_len: int
    anchors: np.ndarray       # [rows] float32 (FP16 values)
    sub_scale: np.ndarray     # [rows, groups] uint8
    indices: np.ndarray       # [rows, vectors] uint16
    sign: np.ndarray          # [rows, groups] uint8: 0 -> +delta (bank 0), 1 -> -delta (bank 1)
    table: np.ndarray | None = None  # L: own [2048, 8] table or None = the grid; S: [2, 512, 8] (None = default banks)

    @property
    def rows(self) -> int:
        return int(self.anchors.size)

    @property
    def nbytes(self) -> int:
        return len(pack_nvq1(self))


def _pack_bits(values: np.ndarray, bits: int) -> bytes:
    v = np.ascontiguousarray(values, dtype=np.uint16).reshape(-1)
    if v.size and int(v.max()) >= (1 << bits):
        raise ValueError(f"value does not fit in {bits} bits")
    rows = ((v[:, None] >> np.arange(bits, dtype=np.uint16)[None, :]) & 1).astype(np.uint8)
    return np.packbits(rows.reshape(-1), bitorder="little").tobytes()


def _unpack_bits(blob, off: int, count: int, bits: int) -> tuple[np.ndarray, int]:
    nbytes = (count * bits + 7) // 8
    if off + nbytes > len(blob):
        raise ValueError("truncated NVQ1 bit stream")
    stream = np.unpackbits(np.frombuffer(blob, dtype=np.uint8, count=nbytes, offset=off), bitorder="little")[: count * bits]
    vals = (stream.reshape(count, bits).astype(np.uint32) << np.arange(bits, dtype=np.uint32)[None, :]).sum(1)
    return vals.astype(np.uint16), off + nbytes


def _check(t: Nvq1Tensor) -> tuple[int, int, int]:
    v = t.variant
    shape = tuple(int(s) for s in t.shape)
    if not shape or not 0 <= t.axis < len(shape):
        raise ValueError(f"invalid NVQ1 shape / axis: {shape}, {t.axis}")
    rows = t.rows
    if int(np.prod(shape)) != rows * t.row_len:
        raise ValueError("NVQ1 shape does not match its rows")
    if v.banked and t.row_len % 8:
        raise ValueError("NVQ1-S rows must be a multiple of 8 long")
    ng, nv = math.ceil(t.row_len / v.groupsize), math.ceil(t.row_len / 8)
    for name, want in (("sub_scale", (rows, ng)), ("indices", (rows, nv)), ("sign", (rows, ng))):
        if np.asarray(getattr(t, name)).shape != want:
            raise ValueError(f"bad {name} shape {np.asarray(getattr(t, name)).shape}, expected {want}")
    if (np.asarray(t.sub_scale) >= (1 << v.sub_bits)).any() or (np.asarray(t.indices) >= v.entries).any() or (np.asarray(t.sign) > 1).any():
        raise ValueError("an NVQ1 code exceeds its packed width")
    with np.errstate(over="ignore", invalid="ignore"):
        a16 = np.asarray(t.anchors, dtype=np.float32).astype(np.float16)
    if not np.isfinite(a16).all() or np.signbit(a16).any():
        raise ValueError("NVQ1 anchors must be finite and non-negative in FP16")
    return rows, ng, nv


def pack_nvq1(t: Nvq1Tensor) -> bytes:
    v = t.variant
    rows, _, _ = _check(t)
    shape = tuple(int(s) for s in t.shape)
    if v.banked:
        banks = v.default_table() if t.table is None else np.asarray(t.table)
        if banks.shape != (2, v.entries, 8):
            raise ValueError("NVQ1-S needs two banks of 512 entries")
        second, table = 1, _pack_table(banks[0], v.entries) + _pack_table(banks[1], v.entries)
    else:
        second, table = (2, _pack_table(t.table, v.entries)) if t.table is not None else (1, b"")
    return b"".join([_HEADER.pack(v.magic, second, v.sub_bits, v.groupsize, t.axis, t.row_len, len(shape)),
                     struct.pack(f"<{len(shape)}q", *shape), struct.pack("<I", rows), table,
                     np.asarray(t.anchors, dtype=np.float32).astype("<f2").tobytes(),
                     _pack_bits(t.sub_scale, v.sub_bits), _pack_bits(t.indices, v.index_bits), _pack_bits(t.sign, 1)])


def unpack_nvq1(blob) -> Nvq1Tensor:
    blob = bytes(blob)
    if len(blob) < _HEADER.size:
        raise ValueError("truncated NVQ1 header")
    magic, second, sub_bits, groupsize, axis, row_len, ndim = _HEADER.unpack_from(blob)
    if magic == b"NQ1L":
        if second not in (1, 2) or groupsize <= 0 or groupsize % 8 or not 1 <= sub_bits <= 8:
            raise ValueError("unsupported NVQ1-L profile")
        v = Nvq1Variant("NVQ1-L", magic, 11, 0.125, False, sub_bits, groupsize)
    elif magic == b"NQ1S":
        if second != 1 or sub_bits != 4 or groupsize != 24 or row_len % 8:
            raise ValueError("unsupported NVQ1-S stream profile")
        v = NVQ1_S
    else:
        raise ValueError(f"not an NVQ1 blob: {magic!r}")
    if ndim <= 0 or row_len <= 0:
        raise ValueError("invalid NVQ1 dimensions")
    off = _HEADER.size
    if off + 8 * ndim + 4 > len(blob):
        raise ValueError("truncated NVQ1 shape")
    shape = tuple(struct.unpack_from(f"<{ndim}q", blob, off))
    off += 8 * ndim
    rows = struct.unpack_from("<I", blob, off)[0]
    off += 4
    table = None
    if v.banked:
        if off + 2048 > len(blob):
            raise ValueError("truncated NVQ1-S tables")
        table = np.stack([_unpack_table(blob[off : off + 1024], 512), _unpack_table(blob[off + 1024 : off + 2048], 512)])
        off += 2048
    elif second == 2:
        if off + 4096 > len(blob):
            raise ValueError("truncated NVQ1-L table")
        table = _unpack_table(blob[off : off + 4096], 2048)
        off += 4096
    if off + 2 * rows > len(blob):
        raise ValueError("truncated NVQ1 anchors")
    anchors = np.frombuffer(blob, dtype="<f2", count=rows, offset=off).astype(np.float32)
    off += 2 * rows
    ng, nv = math.ceil(row_len / v.groupsize), math.ceil(row_len / 8)
    sub, off = _unpack_bits(blob, off, rows * ng, v.sub_bits)
    idx, off = _unpack_bits(blob, off, rows * nv, v.index_bits)
    sign, off = _unpack_bits(blob, off, rows * ng, 1)
    if off != len(blob):
        raise ValueError(f"invalid NVQ1 blob tail: consumed {off} of {len(blob)} bytes")
    t = Nvq1Tensor(v, shape, axis, row_len, anchors, sub.astype(np.uint8).reshape(rows, ng), idx.reshape(rows, nv),
                   sign.astype(np.uint8).reshape(rows, ng), table)
    _check(t)
    return t


def _tables(t: Nvq1Tensor) -> np.ndarray:
    """[2, entries, 8] float32: the table a group uses by its sign bit (the same one twice for NVQ1-L)."""
    v = t.variant
    if v.banked:
        return np.asarray(v.default_table() if t.table is None else t.table, dtype=np.float32)
    one = np.asarray(IQ1S_GRID if t.table is None else t.table, dtype=np.float32)
    return np.stack([one, one])


def dequantize_nvq1(t: Nvq1Tensor) -> np.ndarray:
    v = t.variant
    rows, ng, nv = t.rows, t.sub_scale.shape[1], t.indices.shape[1]
    per = v.groupsize // 8
    vec_sign = np.repeat(t.sign, per, axis=1)[:, :nv]
    code = _tables(t)[vec_sign.astype(np.int64), t.indices.astype(np.int64)]            # [rows, nv, 8]
    code = code + np.where(vec_sign != 0, -v.delta, v.delta).astype(np.float32)[..., None]
    scale = np.repeat(t.anchors[:, None] * t.sub_scale.astype(np.float32), per, axis=1)[:, :nv]
    rec = (code * scale[..., None]).reshape(rows, nv * 8)[:, : t.row_len]
    shape, axis = tuple(t.shape), t.axis
    moved = (shape[axis],) + shape[:axis] + shape[axis + 1 :]
    return np.moveaxis(rec.reshape(moved), 0, axis).astype(np.float32)


# ---- encoder -------------------------------------------------------------------------------------------------------------
def _assign(x, wgt, anchors, tables, v: Nvq1Variant, chunk: int):
    """For fixed row anchors: sub-scale, sign and entries of every group.  x, wgt: [rows, nv, 8] torch; anchors [rows]."""
    import torch
    rows, nv, _ = x.shape
    per = v.groupsize // 8
    ng = math.ceil(nv / per)
    pad = ng * per - nv
    if pad:  # a short last group: empty vectors with zero weight never influence the choice
        x = torch.cat([x, x.new_zeros(rows, pad, 8)], 1)
        wgt = torch.cat([wgt, wgt.new_zeros(rows, pad, 8)], 1)
    qmax = (1 << v.sub_bits) - 1
    best_q = torch.zeros((rows, ng), dtype=torch.int64, device=x.device)
    best_s = torch.zeros_like(best_q)
    best_i = torch.zeros((rows, ng * per), dtype=torch.int64, device=x.device)
    for r0 in range(0, rows, chunk):
        r1 = min(rows, r0 + chunk)
        xv, wv = x[r0:r1].reshape(-1, 8), wgt[r0:r1].reshape(-1, 8)
        a = anchors[r0:r1].repeat_interleave(ng * per)
        err = torch.full(((r1 - r0) * ng,), float("inf"), device=x.device)
        cq = torch.zeros_like(err, dtype=torch.int64)
        cs = torch.zeros_like(cq)
        ci = torch.zeros(((r1 - r0) * ng, per), dtype=torch.int64, device=x.device)
        for sbit, delta in ((0, v.delta), (1, -v.delta)):
            shifted = tables[sbit] + delta                    # [entries, 8]
            cross = (wv * xv) @ shifted.T                      # [vectors, entries]
            quad = wv @ (shifted * shifted).T
            for q in range(qmax + 1):
                s = (a * q)[:, None]
                cost = s * s * quad - 2.0 * s * cross
                val, idx = cost.min(1)
                g_err = val.reshape(-1, per).sum(1)
                better = g_err < err
                err = torch.where(better, g_err, err)
                cq = torch.where(better, torch.full_like(cq, q), cq)
                cs = torch.where(better, torch.full_like(cs, sbit), cs)
                ci = torch.where(better[:, None], idx.reshape(-1, per), ci)
        best_q[r0:r1], best_s[r0:r1], best_i[r0:r1] = cq.reshape(-1, ng), cs.reshape(-1, ng), ci.reshape(r1 - r0, ng * per)
    return best_q, best_s, best_i[:, :nv]


def _basis(q, sbit, idx, tables, v: Nvq1Variant, nv: int):
    """q * (entry + signed delta) per weight: [rows, nv, 8]."""
    import torch
    per = v.groupsize // 8
    vs = sbit.repeat_interleave(per, 1)[:, :nv]
    code = tables[vs, idx] + torch.where(vs != 0, -v.delta, v.delta)[..., None]
    return code * q.repeat_interleave(per, 1)[:, :nv, None].to(code.dtype)


def quantize_nvq1(w, variant="NVQ1-L", *, axis: int = 0, importance=None, iterations: int = 3, table_steps: int = 2,
                  device: str | None = None, chunk_rows: int = 64, train_table: bool = False,
                  validation_fraction: float = 0.125, _fixed_table=None) -> Nvq1Tensor:
    """``w``: any-rank array whose ``axis`` indexes the rows; ``importance [row length]``: optional column weights.

    ``train_table`` (NVQ1-L): also fit a tensor-local 2048-entry ternary table (Lloyd steps from the grid, entries kept
    distinct) on all but every ``1 / validation_fraction``-th row, and keep it -- 4096 more bytes in the blob, profile
    2 -- only if it lowers the error on the held-out rows; otherwise the tensor is encoded with the grid."""
    if train_table and not (VARIANTS[variant] if isinstance(variant, str) else variant).banked:
        return _quantize_with_tensor_table(w, variant, axis=axis, importance=importance, iterations=iterations,
                                           table_steps=max(1, table_steps), device=device, chunk_rows=chunk_rows,
                                           validation_fraction=validation_fraction)
    import torch
    v = VARIANTS[variant] if isinstance(variant, str) else variant
    w = np.asarray(w, dtype=np.float32)
    shape = tuple(w.shape)
    rows_first = np.moveaxis(w, axis, 0).reshape(shape[axis], -1)
    rows, row_len = rows_first.shape
    if v.banked and row_len % 8:
        raise ValueError("NVQ1-S rows must be a multiple of 8 long")
    nv = math.ceil(row_len / 8)
    dev = torch.device(device or "cpu")
    x = torch.zeros((rows, nv * 8), dtype=torch.float32, device=dev)
    x[:, :row_len] = torch.from_numpy(rows_first).to(dev)
    wg = torch.zeros_like(x)
    wg[:, :row_len] = 1.0 if importance is None else torch.as_tensor(np.asarray(importance, dtype=np.float32), device=dev).clamp_min(1e-12)
    x, wg = x.reshape(rows, nv, 8), wg.reshape(rows, nv, 8)
    start = v.default_table() if _fixed_table is None else _fixed_table
    tables = torch.as_tensor(np.asarray(start, dtype=np.float32), device=dev)
    if not v.banked:
        tables = torch.stack([tables, tables])
    qmax = (1 << v.sub_bits) - 1
    # start: the largest group amplitude of a row maps to the top sub-scale
    per = v.groupsize // 8
    amp = x.abs().reshape(rows, -1).max(1).values / (1.0 + v.delta)
    anchors = (amp / qmax).clamp_min(1e-8).half().float()
    q = sbit = idx = None
    for it in range(max(1, iterations)):
        q, sbit, idx = _assign(x, wg, anchors, tables, v, chunk_rows)
        if v.banked and it < table_steps:
            tables = _refit_banks(x, wg, anchors, q, sbit, idx, tables, v)
            q, sbit, idx = _assign(x, wg, anchors, tables, v, chunk_rows)
        basis = _basis(q, sbit, idx, tables, v, nv)
        num, den = (wg * x * basis).sum((1, 2)), (wg * basis * basis).sum((1, 2))
        anchors = torch.where(den > 0, num / den.clamp_min(1e-30), anchors).clamp_min(0).half().float()
        anchors = torch.nan_to_num(anchors, nan=0.0, posinf=65504.0).clamp_max(65504.0)
    q, sbit, idx = _assign(x, wg, anchors, tables, v, chunk_rows)
    table = None
    if v.banked:
        table = tables.round().to(torch.int8).cpu().numpy()
    elif _fixed_table is not None:
        table = np.asarray(_fixed_table, dtype=np.int8)
    return Nvq1Tensor(v, shape, axis, row_len, anchors.cpu().numpy().astype(np.float32), q.cpu().numpy().astype(np.uint8),
                      idx.cpu().numpy().astype(np.uint16), sbit.cpu().numpy().astype(np.uint8), table)


def _refit_banks(x, wg, anchors, q, sbit, idx, tables, v: Nvq1Variant):
    """One Lloyd step on the ternary alphabet: every entry becomes the per-coordinate best of {-1, 0, 1} for the vectors
    assigned to it (in units of their scale, the signed delta removed); entries nobody uses, and duplicates, are re-seeded
    from the grid so that the bank keeps 512 distinct entries."""
    import torch
    rows, nv, _ = x.shape
    per = v.groupsize // 8
    vs = sbit.repeat_interleave(per, 1)[:, :nv]
    s = (anchors[:, None] * q.repeat_interleave(per, 1)[:, :nv].float())
    live = s > 0
    out = []
    levels = torch.tensor([-1.0, 0.0, 1.0], device=x.device)
    for b in (0, 1):
        sel = live & (vs == b)
        delta = v.delta if b == 0 else -v.delta
        xs, ws, ss, ids = x[sel], wg[sel], s[sel][:, None], idx[sel]
        new = tables[b].clone()
        if ids.numel():
            # cost of level l at coordinate c for entry e: sum w (x - s (l + delta))^2  -> choose argmin per (e, c)
            cost = torch.zeros((v.entries, 8, 3), device=x.device)
            for li, l in enumerate(levels):
                cost[:, :, li].index_add_(0, ids, ws * (xs - ss * (l + delta)) ** 2)
            used = torch.zeros(v.entries, dtype=torch.bool, device=x.device)
            used[ids.unique()] = True
            new[used] = levels[cost[used].argmin(-1)]
        # keep entries distinct: duplicates and unused slots take grid entries that are not in the bank yet
        seen, fresh = set(), []
        rows_np = new.round().to(torch.int8).cpu().numpy()
        for e in range(v.entries):
            key = rows_np[e].tobytes()
            if key in seen:
                fresh.append(e)
            else:
                seen.add(key)
        if fresh:
            g = 0
            for e in fresh:
                while IQ1S_GRID[g].tobytes() in seen:
                    g += 1
                rows_np[e] = IQ1S_GRID[g]
                seen.add(IQ1S_GRID[g].tobytes())
            new = torch.as_tensor(rows_np.astype(np.float32), device=x.device)
        out.append(new)
    return torch.stack(out)


def _refit_single_table(x, wg, anchors, q, sbit, idx, table, v: Nvq1Variant):
    """Lloyd step for the one table of NVQ1-L: both signs use it, each with its own delta."""
    import torch
    rows, nv, _ = x.shape
    per = v.groupsize // 8
    vs = sbit.repeat_interleave(per, 1)[:, :nv]
    s = anchors[:, None] * q.repeat_interleave(per, 1)[:, :nv].float()
    live = s > 0
    xs, ws, ss, ids = x[live], wg[live], s[live][:, None], idx[live]
    dl = torch.where(vs[live] != 0, -v.delta, v.delta)[:, None]
    new = table.clone()
    if ids.numel():
        levels = torch.tensor([-1.0, 0.0, 1.0], device=x.device)
        cost = torch.zeros((v.entries, 8, 3), device=x.device)
        for li, l in enumerate(levels):
            cost[:, :, li].index_add_(0, ids, ws * (xs - ss * (l + dl)) ** 2)
        used = torch.zeros(v.entries, dtype=torch.bool, device=x.device)
        used[ids.unique()] = True
        new[used] = levels[cost[used].argmin(-1)]
    rows_np = new.round().to(torch.int8).cpu().numpy()
    seen, fresh = set(), []
    for e in range(v.entries):
        key = rows_np[e].tobytes()
        if key in seen:
            fresh.append(e)
        else:
            seen.add(key)
    if fresh:  # duplicates take unused vectors of the ternary cube, walked in a fixed order
        g = 0
        for e in fresh:
            while True:
                cand = (np.array([(g // 3 ** c) % 3 for c in range(8)], dtype=np.int8) - 1)
                g += 1
                if cand.tobytes() not in seen:
                    break
            rows_np[e] = cand
            seen.add(cand.tobytes())
    return torch.as_tensor(rows_np.astype(np.float32), device=x.device)


def _quantize_with_tensor_table(w, variant, *, axis, importance, iterations, table_steps, device, chunk_rows, validation_fraction):
    import torch
    v = VARIANTS[variant] if isinstance(variant, str) else variant
    w = np.asarray(w, dtype=np.float32)
    rows_first = np.moveaxis(w, axis, 0).reshape(w.shape[axis], -1)
    rows = rows_first.shape[0]
    every = max(2, int(round(1.0 / max(validation_fraction, 1e-6))))
    held = np.arange(rows) % every == every - 1
    if held.all() or not held.any():
        return quantize_nvq1(w, v, axis=axis, importance=importance, iterations=iterations, device=device, chunk_rows=chunk_rows)
    train, valid = rows_first[~held], rows_first[held]
    dev = torch.device(device or "cpu")
    table = np.asarray(IQ1S_GRID, dtype=np.int8)
    for _ in range(table_steps):
        t = quantize_nvq1(train, v, importance=importance, iterations=iterations, device=device, chunk_rows=chunk_rows, _fixed_table=table)
        nv = t.indices.shape[1]
        x = torch.zeros((train.shape[0], nv * 8), dtype=torch.float32, device=dev)
        x[:, : train.shape[1]] = torch.from_numpy(train).to(dev)
        wg = torch.zeros_like(x)
        wg[:, : train.shape[1]] = 1.0 if importance is None else torch.as_tensor(np.asarray(importance, dtype=np.float32), device=dev).clamp_min(1e-12)
        new = _refit_single_table(x.reshape(-1, nv, 8), wg.reshape(-1, nv, 8), torch.from_numpy(t.anchors).to(dev),
                                  torch.from_numpy(t.sub_scale.astype(np.int64)).to(dev), torch.from_numpy(t.sign.astype(np.int64)).to(dev),
                                  torch.from_numpy(t.indices.astype(np.int64)).to(dev), torch.as_tensor(table.astype(np.float32), device=dev), v)
        table = new.round().to(torch.int8).cpu().numpy()

    def held_error(tab):
        t = quantize_nvq1(valid, v, importance=importance, iterations=iterations, device=device, chunk_rows=chunk_rows, _fixed_table=tab)
        d = dequantize_nvq1(t) - valid
        return float((d * d * (1.0 if importance is None else np.asarray(importance, dtype=np.float32))).sum())

    if held_error(table) < held_error(None):
        return quantize_nvq1(w, v, axis=axis, importance=importance, iterations=iterations, device=device, chunk_rows=chunk_rows,
                             _fixed_table=table)
    return quantize_nvq1(w, v, axis=axis, importance=importance, iterations=iterations, device=device, chunk_rows=chunk_rows)
