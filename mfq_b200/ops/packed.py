"""Run-time layout of packed expert weights (NINT 1..8 bit, MXFP4) and the kernels that multiply them without ever
expanding them in HBM (``csrc/packed_gemv.cu``).

The checkpoint keeps a tensor's codes as bit streams (``formats/nint.py``, ``formats/mx.py``).  At load time the SAME
codes are re-arranged -- rows sorted by code width into 16-row tiles, inputs cut into 128-code units, every code split
into 4/2/1-bit planes laid out so that a thread's share of a unit is a few aligned words -- which is what lets the
kernel turn a pair of codes into two bf16 numbers with one shift and one logic operation.  Nothing is re-quantized:
:func:`dequantize` rebuilds exactly the matrix ``formats.nint.dequantize_nint_rows`` / ``formats.mx.dequantize_mx``
give (the kernel then evaluates ``q * s - m`` in bf16 arithmetic).

The reference keeps per-projection run-time payloads behind a 184-byte descriptor as well
(``mfq/kernels/cuda/mfe_ffn.h:9-41``); its decode kernels are dp4a kernels over int8-quantized activations.
"""

from __future__ import annotations

import ctypes as C
import math
from dataclasses import dataclass

import numpy as np
import torch

from .lib import check, lib, ptr, stream_ptr

MXFP4_BITS = 16  # width code of an MXFP4 tile in ``tile_meta`` (NINT tiles carry their code width, 1..8)
UNIT = 128


def _planes(bits: int) -> list[tuple[int, int]]:
    """(plane width, right shift of the code) of every plane of a ``bits``-wide code, in storage order."""
    if bits == MXFP4_BITS:
        return [(4, 0)]
    if bits == 8:
        return [(4, 0), (4, 4)]
    out, sh = [], 0
    for p in (4, 2, 1):
        if bits & p:
            out.append((p, sh))
            sh += p
    return out


def words_per_thread(bits: int) -> int:
    return 4 if bits == MXFP4_BITS else bits


def _pack_plane(vals: np.ndarray, p: int) -> np.ndarray:
    """``vals [..., 32]`` plane values (< 2**p) of a thread's 32 consecutive codes -> ``[..., p]`` uint32 words: code
    ``2 i + h`` of the run goes to word ``i // (16 // p)`` at bit ``p * (i % (16 // p)) + 16 h``."""
    per = 16 // p  # pairs per word
    v = vals.astype(np.uint32).reshape(*vals.shape[:-1], 16, 2)  # [..., pair, half]
    words = np.zeros((*vals.shape[:-1], p), dtype=np.uint32)
    for i in range(16):
        sh = p * (i % per)
        words[..., i // per] |= (v[..., i, 0] << np.uint32(sh)) | (v[..., i, 1] << np.uint32(sh + 16))
    return words


def _unpack_plane(words: np.ndarray, p: int) -> np.ndarray:
    per = 16 // p
    out = np.zeros((*words.shape[:-1], 32), dtype=np.uint8)
    mask = np.uint32((1 << p) - 1)
    for i in range(16):
        sh = p * (i % per)
        w = words[..., i // per]
        out[..., 2 * i] = (w >> np.uint32(sh)) & mask
        out[..., 2 * i + 1] = (w >> np.uint32(sh + 16)) & mask
    return out


@dataclass
class PackedMatrix:
    """One ``[n_out, k_in]`` matrix in the run-time layout (host arrays)."""

    n_out: int
    k_in: int
    gs: int  # NINT group size (16, 24 or 32); MXFP4: 32
    units: int
    g4: int
    tile_bits: np.ndarray  # [tiles] int32
    tile_off: np.ndarray  # [tiles] int32 word offset of the tile's codes
    tile_goff: np.ndarray  # [tiles] int32 byte offset of the tile's group parameters
    tile_gs: np.ndarray  # [tiles] int32 NINT group size of the tile (32 for MXFP4)
    codes: np.ndarray  # uint32 words
    gparams: np.ndarray  # uint8
    anchors: np.ndarray  # [tiles*16, 2] float16 (d, dmin); zeros for MXFP4
    out_row: np.ndarray  # [tiles*16] int32

    @property
    def tiles(self) -> int:
        return int(self.tile_bits.shape[0])

    def nbytes(self) -> int:
        return self.codes.nbytes + self.gparams.nbytes + self.anchors.nbytes + self.out_row.nbytes + 8 * self.tiles

    def bits_per_weight(self) -> float:
        return 8.0 * self.nbytes() / (self.n_out * self.k_in)


def _tile_rows(widths: np.ndarray) -> tuple[np.ndarray, np.ndarray]:
    """Rows sorted by code width and cut into 16-row tiles of one width: (tile widths, ``[tiles, 16]`` row ids, -1 pad)."""
    bits, rows = [], []
    for b in sorted(set(int(w) for w in widths)):
        idx = np.flatnonzero(widths == b)
        pad = (-idx.size) % 16
        idx = np.concatenate([idx, np.full(pad, -1, dtype=np.int64)]).reshape(-1, 16)
        rows.append(idx)
        bits += [b] * idx.shape[0]
    return np.asarray(bits, dtype=np.int32), np.concatenate(rows, 0)


def _group_words(units: int, gs: int) -> int:
    """4-group parameter words per row that the kernel's indexing can reach."""
    return units if gs == 32 else units * 2 if gs == 16 else (units * 4 - 1) // 3 + 1


def nint_units(t) -> int:
    return math.ceil(t.groups * int(t.spec.groupsize) / UNIT)


def pack_nint(t, min_units: int = 0) -> PackedMatrix:
    """:class:`~mfq_b200.formats.nint.NintTensor` (quantized along its last logical axis) -> run-time layout.
    ``min_units``: pad the input range to at least this many 128-code units (experts of a projection share it)."""
    gs = int(t.spec.groupsize)
    if gs not in (16, 24, 32):
        raise ValueError(f"the packed kernels take NINT group sizes 16, 24 and 32, not {gs}")
    n, groups = t.out, t.groups
    k_codes = groups * gs
    units = max(min_units, math.ceil(k_codes / UNIT))
    g4 = _group_words(units, gs)
    q = np.zeros((n, units * UNIT), dtype=np.uint8)
    q[:, :k_codes] = t.q.reshape(n, k_codes)
    ls = np.zeros((n, g4 * 4), dtype=np.uint8)
    lm = np.zeros((n, g4 * 4), dtype=np.uint8)
    ls[:, :groups], lm[:, :groups] = t.sub_scale, t.sub_min
    tile_bits, tile_rows = _tile_rows(t.q_widths())
    tiles = tile_bits.shape[0]
    safe = np.where(tile_rows < 0, 0, tile_rows)
    live = (tile_rows >= 0)
    # [tiles, 16, units, 4 threads, 32 codes]
    qt = (q[safe] * live[..., None]).reshape(tiles, 16, units, 4, 32)
    chunks, offs, off = [], [], 0
    for ti in range(tiles):
        b = int(tile_bits[ti])
        offs.append(off)
        per_unit = []
        for p, sh in _planes(b):
            vals = (qt[ti] >> sh) & ((1 << p) - 1)  # [16, units, 4, 32]
            words = _pack_plane(vals, p)  # [16, units, 4, p]
            per_unit.append(words.transpose(1, 0, 2, 3).reshape(units, 64 * p))  # [units][row 16][thread 4][p]
        tile_words = np.concatenate(per_unit, axis=1).reshape(-1)  # [units][planes...]
        chunks.append(tile_words)
        off += tile_words.size
    gp = np.zeros((tiles * 16, g4, 2, 4), dtype=np.uint8)
    gp[:, :, 0, :] = (ls[safe] * live[..., None]).reshape(tiles * 16, g4, 4)
    gp[:, :, 1, :] = (lm[safe] * live[..., None]).reshape(tiles * 16, g4, 4)
    anchors = np.zeros((tiles * 16, 2), dtype=np.float16)
    anchors[:, 0] = (np.asarray(t.neuron_scale, dtype=np.float32)[safe] * live).reshape(-1)
    anchors[:, 1] = (np.asarray(t.neuron_min, dtype=np.float32)[safe] * live).reshape(-1)
    return PackedMatrix(n, int(t.neuron_len), gs, units, g4, tile_bits, np.asarray(offs, dtype=np.int32),
                        (np.arange(tiles) * 16 * g4 * 8).astype(np.int32), np.full(tiles, gs, dtype=np.int32),
                        np.concatenate(chunks).astype(np.uint32), gp.reshape(-1), anchors, tile_rows.reshape(-1).astype(np.int32))


def pack_mxfp4(t, min_units: int = 0) -> PackedMatrix:
    """:class:`~mfq_b200.formats.mx.MxTensor` of kind MXFP4 -> run-time layout (every tile has width code 16)."""
    n, k = (int(v) for v in t.shape)
    units = max(min_units, math.ceil(k / UNIT))
    vals = np.asarray(t.values, dtype=np.uint8)
    codes = np.zeros((n, units * UNIT), dtype=np.uint8)
    codes[:, 0:k:2] = vals & 0xF
    codes[:, 1:k:2] = vals >> 4
    scales = np.zeros((n, units * 4), dtype=np.uint8)
    scales[:, : k // 32] = np.asarray(t.scales, dtype=np.uint8)
    tile_bits, tile_rows = _tile_rows(np.full(n, MXFP4_BITS))
    tiles = tile_bits.shape[0]
    safe, live = np.where(tile_rows < 0, 0, tile_rows), tile_rows >= 0
    qt = (codes[safe] * live[..., None]).reshape(tiles, 16, units, 4, 32)
    words = _pack_plane(qt, 4)  # [tiles, 16, units, 4, 4]
    code_words = words.transpose(0, 2, 1, 3, 4).reshape(tiles, -1)
    gp = (scales[safe] * live[..., None]).reshape(tiles * 16, units, 4)
    return PackedMatrix(n, k, 32, units, units, tile_bits, (np.arange(tiles) * code_words.shape[1]).astype(np.int32),
                        (np.arange(tiles) * 16 * units * 4).astype(np.int32), np.full(tiles, 32, dtype=np.int32),
                        code_words.reshape(-1).astype(np.uint32), gp.reshape(-1), np.zeros((tiles * 16, 2), dtype=np.float16),
                        tile_rows.reshape(-1).astype(np.int32))


def dequantize(m: PackedMatrix) -> np.ndarray:
    """fp32 ``[n_out, k_in]`` matrix of a packed layout, in exact arithmetic (the oracle of the kernels)."""
    from ..formats.mx import E2M1_VALUES
    out = np.zeros((m.n_out, m.k_in), dtype=np.float32)
    rows = m.out_row.reshape(m.tiles, 16)
    for ti in range(m.tiles):
        b = int(m.tile_bits[ti])
        wpt = words_per_thread(b)
        block = m.codes[m.tile_off[ti] : m.tile_off[ti] + m.units * 64 * wpt].reshape(m.units, 64 * wpt)
        code = np.zeros((16, m.units, 4, 32), dtype=np.uint16)
        o = 0
        for p, sh in _planes(b):
            words = block[:, o : o + 64 * p].reshape(m.units, 16, 4, p).transpose(1, 0, 2, 3)
            code |= _unpack_plane(words, p).astype(np.uint16) << sh
            o += 64 * p
        code = code.reshape(16, m.units * UNIT)
        g0 = int(m.tile_goff[ti])
        if b == MXFP4_BITS:
            sc = m.gparams[g0 : g0 + 16 * m.units * 4].reshape(16, m.units * 4)
            mag = E2M1_VALUES[code & 7] * np.where(code & 8, -1.0, 1.0)
            w = mag * np.repeat(np.ldexp(np.float32(1.0), sc.astype(np.int32) - 127), 32, axis=1)
        else:
            gs = int(m.tile_gs[ti])
            g4 = _group_words(m.units, gs)
            gp = m.gparams[g0 : g0 + 16 * g4 * 8].reshape(16, g4, 2, 4)
            ls = gp[:, :, 0, :].reshape(16, -1).astype(np.float32)
            lm = gp[:, :, 1, :].reshape(16, -1).astype(np.float32)
            an = m.anchors[ti * 16 : ti * 16 + 16].astype(np.float32)
            g = np.arange(m.units * UNIT) // gs
            w = code.astype(np.float32) * (an[:, :1] * ls[:, g]) - an[:, 1:] * lm[:, g]
        for r in range(16):
            if rows[ti, r] >= 0:
                out[rows[ti, r]] = w[r, : m.k_in]
    return out


def concat_rows(parts: list[PackedMatrix]) -> PackedMatrix:
    """Matrices over the same inputs stacked along the output features (gate on top of up): tiles are simply listed one
    after the other, so the parts may differ in family and width."""
    first = parts[0]
    if any((m.k_in, m.units) != (first.k_in, first.units) for m in parts):
        raise ValueError("stacked matrices must share their (padded) input range")
    rows, coff, goff = 0, 0, 0
    tile_off, tile_goff, out_row = [], [], []
    for m in parts:
        tile_off.append(m.tile_off + coff)
        tile_goff.append(m.tile_goff + goff)
        out_row.append(np.where(m.out_row >= 0, m.out_row + rows, -1))
        rows, coff, goff = rows + m.n_out, coff + m.codes.size, goff + (m.gparams.size + 15) // 16 * 16
    gbuf = np.zeros(goff, dtype=np.uint8)
    g0 = 0
    for m in parts:
        gbuf[g0 : g0 + m.gparams.size] = m.gparams
        g0 += (m.gparams.size + 15) // 16 * 16
    return PackedMatrix(rows, first.k_in, first.gs, first.units, first.g4,
                        np.concatenate([m.tile_bits for m in parts]), np.concatenate(tile_off).astype(np.int32),
                        np.concatenate(tile_goff).astype(np.int32), np.concatenate([m.tile_gs for m in parts]),
                        np.concatenate([m.codes for m in parts]), gbuf,
                        np.concatenate([m.anchors for m in parts]), np.concatenate(out_row).astype(np.int32))


def _expert_slice(tensor, pos: int, out: int):
    """Rows ``[pos * out, (pos + 1) * out)`` of a pool's stacked family tensor, as a tensor of the same family (or None
    when the family has no packed kernel)."""
    from ..formats.mx import MXFP4_DTYPE, MxTensor
    from ..formats.mxfp4sq import Mxfp4SqTensor, expanded
    from ..formats.nint import NintTensor
    if isinstance(tensor, Mxfp4SqTensor):
        tensor = expanded(tensor)  # every palette-coded row is a legal MXFP4 row
    r = slice(pos * out, (pos + 1) * out)
    if isinstance(tensor, NintTensor) and int(tensor.spec.groupsize) in (16, 24, 32) and tensor.axis == 0:
        return NintTensor(spec=tensor.spec, shape=(out, tensor.neuron_len), axis=0, neuron_len=tensor.neuron_len, q=tensor.q[r],
                          neuron_scale=tensor.neuron_scale[r], neuron_min=tensor.neuron_min[r], sub_scale=tensor.sub_scale[r],
                          sub_min=tensor.sub_min[r], row_q_bits=None if tensor.row_q_bits is None else tensor.row_q_bits[r],
                          row_sub_bits=None if tensor.row_sub_bits is None else tensor.row_sub_bits[r])
    if isinstance(tensor, MxTensor) and tensor.dtype == MXFP4_DTYPE:
        return MxTensor(MXFP4_DTYPE, (out, tensor.shape[1]), np.asarray(tensor.values)[r], np.asarray(tensor.scales)[r])
    return None


def expert_units(mfe, experts) -> int | None:
    """128-code units that every packed expert of ``mfe`` needs (None: some expert's family has no packed kernel)."""
    from ..formats.nint import NintTensor
    where = mfe.expert_location()
    units = 0
    for e in experts:
        pi, pos = where[int(e)]
        t = _expert_slice(mfe.pools[pi].tensor, pos, mfe.shape[1])
        if t is None:
            return None
        units = max(units, nint_units(t) if isinstance(t, NintTensor) else math.ceil(t.shape[1] / UNIT))
    return units


def pack_expert(mfe, expert: int, min_units: int) -> PackedMatrix:
    from ..formats.nint import NintTensor
    pi, pos = mfe.expert_location()[int(expert)]
    t = _expert_slice(mfe.pools[pi].tensor, pos, mfe.shape[1])
    return pack_nint(t, min_units) if isinstance(t, NintTensor) else pack_mxfp4(t, min_units)


def pack_moe_projection(parts, experts, device) -> "PackedExperts | None":
    """``parts``: the MFE tensors stacked along the output features (``[gate, up]`` or ``[down]``); returns the packed
    experts ``experts`` of that projection, or None when a family without a packed kernel (NVQ, FP8, float) occurs."""
    from ..formats.mfe import MfeTensor
    if not all(isinstance(p, MfeTensor) for p in parts):
        return None
    units = [expert_units(p, experts) for p in parts]
    if any(u is None for u in units):
        return None
    u = max(units)
    try:
        return PackedExperts([concat_rows([pack_expert(p, e, u) for p in parts]) for e in experts], device)
    except ValueError:
        return None


class PackedExperts:
    """The matrices of one projection of ``E`` experts on the device, as the kernels address them."""

    def __init__(self, mats: list[PackedMatrix], device) -> None:
        first = mats[0]
        if any((m.n_out, m.k_in, m.units) != (first.n_out, first.k_in, first.units) for m in mats):
            raise ValueError("the experts of a projection must share shape and padded input range (see min_units)")
        self.n_out, self.k_in, self.units = first.n_out, first.k_in, first.units
        self.experts = len(mats)
        self.tiles = max(m.tiles for m in mats)
        t16 = self.tiles * 16
        meta = np.zeros((self.experts, self.tiles, 4), dtype=np.int32)
        anchors = np.zeros((self.experts, t16, 2), dtype=np.float16)
        out_row = np.full((self.experts, t16), -1, dtype=np.int32)
        code_base, gparam_base, cpos, gpos = [], [], 0, 0
        for e, m in enumerate(mats):
            meta[e, : m.tiles, 0], meta[e, : m.tiles, 1], meta[e, : m.tiles, 2] = m.tile_bits, m.tile_off, m.tile_goff
            meta[e, : m.tiles, 3] = m.tile_gs
            anchors[e, : m.tiles * 16], out_row[e, : m.tiles * 16] = m.anchors, m.out_row
            code_base.append(cpos)
            gparam_base.append(gpos)
            cpos += m.codes.size
            gpos += (m.gparams.size + 15) // 16 * 16
        gbuf = np.zeros(gpos, dtype=np.uint8)
        for m, g0 in zip(mats, gparam_base):
            gbuf[g0 : g0 + m.gparams.size] = m.gparams
        dev = torch.device(device)
        self.codes = torch.from_numpy(np.concatenate([m.codes for m in mats]).view(np.int32)).to(dev)
        self.code_base = torch.tensor(code_base, dtype=torch.int64, device=dev)
        self.tile_meta = torch.from_numpy(meta).to(dev)
        self.gparams = torch.from_numpy(gbuf).to(dev)
        self.gparam_base = torch.tensor(gparam_base, dtype=torch.int64, device=dev)
        self.anchors = torch.from_numpy(anchors).to(dev)
        self.out_row = torch.from_numpy(out_row).to(dev)

    @classmethod
    def synthetic(cls, experts: int, n_out: int, k_in: int, bits, device, gs: int = 32, seed: int = 0, std: float = 0.02):
        """Structurally valid random payloads generated on the device (performance fixtures for models whose real
        quantization would take hours): ``bits`` is one width code per expert (1..8 NINT, 16 MXFP4); all rows of an
        expert share it.  Codes, group codes and anchors are drawn so that weights come out with about ``std``."""
        self = cls.__new__(cls)
        dev = torch.device(device)
        gen = torch.Generator(device=dev).manual_seed(seed)
        self.n_out, self.k_in, self.experts = n_out, k_in, experts
        self.units = math.ceil(math.ceil(k_in / gs) * gs / UNIT)
        g4 = _group_words(self.units, gs)
        self.tiles = math.ceil(n_out / 16)
        bits = [int(b) for b in bits]
        assert len(bits) == experts and n_out % 16 == 0
        wpt = torch.tensor([words_per_thread(b) for b in bits], dtype=torch.int64)
        words_per_expert = self.tiles * self.units * 64 * wpt
        code_base = torch.cumsum(words_per_expert, 0) - words_per_expert
        total = int(words_per_expert.sum())
        self.codes = torch.randint(-2 ** 31, 2 ** 31 - 1, (total,), generator=gen, device=dev, dtype=torch.int32)
        self.code_base = code_base.to(dev)
        meta = torch.zeros((experts, self.tiles, 4), dtype=torch.int32)
        meta[:, :, 0] = torch.tensor(bits, dtype=torch.int32)[:, None]
        meta[:, :, 1] = (torch.arange(self.tiles)[None, :] * (self.units * 64 * wpt)[:, None]).to(torch.int32)
        t16 = self.tiles * 16
        per_tile = torch.tensor([16 * (self.units * 4 if b == MXFP4_BITS else g4 * 8) for b in bits], dtype=torch.int64)
        meta[:, :, 2] = (torch.arange(self.tiles)[None, :] * per_tile[:, None]).to(torch.int32)
        meta[:, :, 3] = gs
        self.tile_meta = meta.to(dev)
        gbytes = per_tile * self.tiles
        self.gparam_base = (torch.cumsum(gbytes, 0) - gbytes).to(dev)
        # group codes: NINT ls / lm in 32..63 (six-bit codes); MXFP4 scale exponents around 2^-6
        gp = torch.randint(32, 64, (int(gbytes.sum()),), generator=gen, device=dev, dtype=torch.int32).to(torch.uint8)
        for e, b in enumerate(bits):
            if b == MXFP4_BITS:
                g0 = int(self.gparam_base[e])
                gp[g0 : g0 + int(gbytes[e])] = 127 - 7
        self.gparams = gp
        # w = d ls q - dmin lm with q uniform in [0, 2^b): centre it and give it the requested spread
        anchors = torch.zeros((experts, t16, 2), dtype=torch.float16)
        for e, b in enumerate(bits):
            if b != MXFP4_BITS:
                qmax = (1 << b) - 1
                d = std * math.sqrt(12.0) / (48.0 * (qmax + 1))
                anchors[e, :, 0], anchors[e, :, 1] = d, d * qmax / 2.0
        self.anchors = anchors.to(dev)
        self.out_row = torch.arange(n_out, dtype=torch.int32, device=dev).repeat(experts, 1)
        return self

    def nbytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.codes, self.gparams, self.anchors, self.out_row, self.tile_meta))

    def bits_per_weight(self) -> float:
        return 8.0 * self.nbytes() / (self.experts * self.n_out * self.k_in)

    def _args(self):
        return (ptr(self.codes), ptr(self.code_base), ptr(self.tile_meta), ptr(self.gparams), ptr(self.gparam_base),
                ptr(self.anchors), ptr(self.out_row), self.tiles, self.units)

    def dense(self, expert: int) -> torch.Tensor:
        """bf16 ``[n_out, k_in]`` reconstruction of one expert by the GPU decode routines."""
        out = torch.zeros((self.n_out, self.k_in + self.k_in % 2), dtype=torch.bfloat16, device=self.codes.device)
        fn = lib().mfq_packed_dequant
        fn.restype = C.c_int
        fn.argtypes = [C.c_void_p] * 7 + [C.c_int] * 3 + [C.c_void_p, C.c_int, C.c_void_p]
        check(fn(*self._args(), expert, ptr(out), out.shape[1], stream_ptr()), "packed_dequant")
        return out[:, : self.k_in]


def packed_gemv_grouped(w: PackedExperts, x: torch.Tensor, plan, gather: bool) -> torch.Tensor:
    """``out[sorted row] = W_expert(row) @ x[row]`` for every route of ``plan`` (token tile 16).  ``x``: bf16 ``[T, K]``
    token rows with ``gather`` (read through the plan's row -> token map), else the expert-sorted rows."""
    assert plan.token_tile == 16 and x.dtype == torch.bfloat16 and x.stride(1) == 1
    out = torch.empty((plan.max_rows, w.n_out), dtype=torch.bfloat16, device=x.device)
    fn = lib().mfq_packed_gemv_grouped
    fn.restype = C.c_int
    fn.argtypes = [C.c_void_p] * 7 + [C.c_int] * 2 + [C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_int, C.c_void_p, C.c_int,
                                                      C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]
    tokens = plan.dest.shape[0]  # an expert receives each token at most once
    rc = fn(*w._args(), ptr(x), x.stride(0), min(w.k_in, x.shape[1]), ptr(out), w.n_out, ptr(plan.tile_map),
            plan.tile_map.shape[0], ptr(plan.offsets), ptr(plan.src_token) if gather else None, tokens, stream_ptr())
    check(rc, "packed_gemv_grouped")
    return out


def moe_ffn_packed(x: torch.Tensor, topk_ids: torch.Tensor, topk_w: torch.Tensor, gate_up: PackedExperts,
                   down: PackedExperts, *, e_lo: int = 0, base=None, extra=None, out=None) -> torch.Tensor:
    """Routed experts of one layer over packed weights: ``base + extra + sum_k w * expert_k(x)`` with ``x`` the
    normalized bf16 activations.  Gate/up product (gather folded into the loads), SwiGLU, down product, weighted
    un-permute; every product decodes its weights in registers."""
    from . import kernels as K
    from . import moe
    plan = moe.plan_routes(topk_ids, e_lo, e_lo + gate_up.experts, token_tile=16)
    gu = packed_gemv_grouped(gate_up, x, plan, gather=True)
    h = K.silu_mul(gu)
    y = packed_gemv_grouped(down, h, plan, gather=False)
    return moe.combine(y, plan, topk_w, base, extra, out)
