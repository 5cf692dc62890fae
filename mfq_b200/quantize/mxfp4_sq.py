"""MXFP4-SQ palette quantizer: re-code a native MXFP4 matrix at 1-3 bits per weight without leaving the MXFP4 value set.

A compressed row keeps ``q``-bit symbols and eight STATES; a state is a catalogue palette (``2**q`` E2M1 values) and one
of four block exponents ``base .. base + 3`` (``base`` is shared by the matrix).  A block of 32 weights picks its state
with one stored bit and two bits that ride in the XOR of its symbols (``formats/mxfp4sq.py``), and decodes to ordinary
E2M1 nibbles under an ordinary E8M0 scale, so the result still runs on the MXFP4 tensor-core path.

The search, per row and width ``q`` (all of it table lookups over the 16 nibble values, no floating-point rounding):

1. ``cost[e, d, p, n, l]``: squared error of coding nibble ``n`` of a block with source exponent ``base + e`` by level
   ``l`` of palette ``p`` under exponent ``base + d``.  Its minimum over ``l`` summed with a block's nibble histogram is
   that block's error under candidate state ``(p, d)`` -- one small matrix product per distinct source exponent.
2. Eight of the 128 candidates are chosen for the row by greedy facility location on the block-by-candidate error
   matrix, followed by one exchange pass (each slot re-chosen with the other seven fixed) and two Lloyd rounds.
3. Every block takes the state with the least error INCLUDING the price of steering the symbol XOR to that state's low
   two bits: either one symbol moves to the level whose index differs by the required XOR, or two symbols share it;
   the cheapest of those repairs is found from the two smallest penalties per XOR value (for ``q = 1`` the tag bits are
   the parities of the even and odd lanes, each fixed by flipping the cheapest lane of that parity).

Rows are given their width from a mean-bits target by the usual greedy exchange: start every row at ``q = 4`` (lossless)
and repeatedly narrow the row that adds the least error per byte saved.

Reference: ``mfq/quantize/mxfp4_sq.py:287-308`` (exponent window), ``:311-338,341-413`` (tables, tag repair),
``:476-750`` (row states), ``:849-929`` (public entry point).
"""

from __future__ import annotations

import heapq

import numpy as np

from ..formats.bitstream import pack_bits
from ..formats.mx import MXFP4_DTYPE, MxTensor
from ..formats.mxfp4sq import PALETTES, Mxfp4SqTensor, block_tags

__all__ = ["quantize_mxfp4_sq", "row_nbytes", "select_scale_base"]

_VAL = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, 0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0], dtype=np.float64)
# required XOR r -> the pair (a, b) with a ^ b = r that two symbols can share
_PAIR = {1: (2, 3), 2: (1, 3), 3: (1, 2)}


def row_nbytes(q: int, cols: int) -> int:
    """Bytes a row of width ``q`` occupies in the container (symbols + its share of the side streams; the bit-packed
    side streams are counted at their exact fractional size rounded up per row, a bound that is tight to a byte)."""
    blocks = cols // 32
    return cols // 2 + blocks if q == 4 else cols * q // 8 + (blocks + 7) // 8 + 2 + 5


def select_scale_base(nibbles: np.ndarray, scales: np.ndarray) -> int:
    """The four-exponent window ``[base, base + 3]`` that loses the least energy when block exponents are clamped to it."""
    energy = (_VAL[nibbles] ** 2).reshape(scales.shape[0], scales.shape[1], 32).sum(-1)
    s = scales.astype(np.int64)
    best = None
    for base in range(max(0, int(s.min()) - 3), min(251, int(s.max())) + 1):
        clipped = np.clip(s, base, base + 3)
        loss = float((energy * (np.exp2((s - 127).astype(np.float64)) - np.exp2((clipped - 127).astype(np.float64))) ** 2).sum())
        key = (loss, abs(base - int(s.min())), base)
        if best is None or key < best:
            best = key
    return int(best[2])


def _cost_table(q: int, e_lo: int, e_hi: int) -> np.ndarray:
    """``[e_hi - e_lo + 1, 4, 32, 16, 2**q]`` float64, in units of ``2**(2 * (base - 127))``."""
    levels = _VAL[PALETTES[q]]                                                         # [32, L]
    e = np.arange(e_lo, e_hi + 1, dtype=np.float64)
    src = _VAL[None, :] * np.exp2(e)[:, None]                                          # [E, 16]
    rec = levels[None, :, :] * np.exp2(np.arange(4, dtype=np.float64))[:, None, None]  # [4, 32, L]
    return (src[:, None, None, :, None] - rec[None, :, :, None, :]) ** 2


def _choose_states(err: np.ndarray) -> np.ndarray:
    """``err [R, B, C]`` -> ``[R, 8]`` candidate ids: greedy facility location, then one exchange pass."""
    r, b, c = err.shape
    chosen = np.zeros((r, 8), dtype=np.int64)
    cur = np.full((r, b), np.inf)
    rows = np.arange(r)
    for k in range(8):
        total = np.minimum(cur[:, :, None], err).sum(1)                                # [R, C]
        chosen[:, k] = total.argmin(1)
        cur = np.minimum(cur, err[rows, :, chosen[:, k]])
    for k in range(8):
        others = np.full((r, b), np.inf)
        for j in range(8):
            if j != k:
                others = np.minimum(others, err[rows, :, chosen[:, j]])
        chosen[:, k] = np.minimum(others[:, :, None], err).sum(1).argmin(1)
    for _ in range(2):  # Lloyd: blocks to their nearest state, every state to the best candidate for its blocks
        mine = np.stack([err[rows, :, chosen[:, k]] for k in range(8)], -1).argmin(-1)          # [R, B]
        for k in range(8):
            load = ((mine == k)[:, :, None] * err).sum(1)                                        # [R, C]
            used = (mine == k).any(1)
            chosen[:, k] = np.where(used, load.argmin(1), chosen[:, k])
    return chosen


def _two_smallest(pen: np.ndarray):
    """Along the last axis: (smallest, its index, second smallest)."""
    i1 = pen.argmin(-1)
    m1 = np.take_along_axis(pen, i1[..., None], -1)[..., 0]
    masked = pen.copy()
    np.put_along_axis(masked, i1[..., None], np.inf, -1)
    return m1, i1, masked.min(-1), masked.argmin(-1)


def _encode_rows(nib: np.ndarray, scales: np.ndarray, q: int, base: int, table: np.ndarray, e_lo: int):
    """Rows of one width.  ``nib [R, B, 32]``, ``scales [R, B]``.  Returns (symbols [R, B, 32], selectors [R, B],
    state scales [R, 8], state palettes [R, 8], row errors [R])."""
    r, b, _ = nib.shape
    levels = 1 << q
    e_idx = np.clip(scales.astype(np.int64) - base, e_lo, e_lo + table.shape[0] - 1) - e_lo     # [R, B]
    best = table.min(-1)                                                                       # [E, 4, 32, 16]
    hist = (nib[..., None] == np.arange(16, dtype=np.uint8)).sum(2).astype(np.float64)         # [R, B, 16]
    err = np.empty((r, b, 128))
    for e in np.unique(e_idx):
        where = e_idx == e
        err[where] = hist[where] @ best[e].reshape(128, 16).T                                  # candidate = d * 32 + p
    chosen = _choose_states(err)                                                               # [R, 8]
    d_of, p_of = chosen // 32, chosen % 32
    # cost of every level for every lane under each of the row's eight states: [R, B, 8, 32, L]
    lane = table[e_idx[:, :, None, None], d_of[:, None, :, None], p_of[:, None, :, None], nib[:, :, None, :].astype(np.int64)]
    sym = lane.argmin(-1)                                                                      # [R, B, 8, 32]
    floor = np.take_along_axis(lane, sym[..., None], -1)[..., 0]
    total = floor.sum(-1)                                                                      # [R, B, 8]
    want = (np.arange(8) & 3)[None, None, :]
    if q == 1:
        other = np.take_along_axis(lane, (sym ^ 1)[..., None], -1)[..., 0] - floor             # price of flipping a lane
        tag = np.bitwise_xor.reduce(sym[..., 0::2], axis=-1) | (np.bitwise_xor.reduce(sym[..., 1::2], axis=-1) << 1)
        need = tag ^ want
        even_i, odd_i = other[..., 0::2].argmin(-1) * 2, other[..., 1::2].argmin(-1) * 2 + 1
        even_c = np.take_along_axis(other, even_i[..., None], -1)[..., 0]
        odd_c = np.take_along_axis(other, odd_i[..., None], -1)[..., 0]
        total = total + np.where(need & 1, even_c, 0.0) + np.where(need & 2, odd_c, 0.0)
        state = total.argmin(-1)                                                               # [R, B]
        pick = lambda a: np.take_along_axis(a, state[..., None], 2)[:, :, 0]
        out = np.take_along_axis(sym, state[..., None, None], 2)[:, :, 0, :].copy()
        need_s, ei, oi = pick(need), pick(even_i), pick(odd_i)
        rr, bb = np.nonzero(need_s & 1)
        out[rr, bb, ei[rr, bb]] ^= 1
        rr, bb = np.nonzero(need_s & 2)
        out[rr, bb, oi[rr, bb]] ^= 1
    else:
        tag = np.bitwise_xor.reduce(sym & 3, axis=-1)
        need = tag ^ want                                                                      # [R, B, 8] in 0..3
        pen = {x: np.take_along_axis(lane, (sym ^ x)[..., None], -1)[..., 0] - floor for x in (1, 2, 3)}
        small = {x: _two_smallest(pen[x]) for x in (1, 2, 3)}
        repair_cost = np.zeros(need.shape)
        plan = np.zeros(need.shape + (4,), dtype=np.int64)          # lane a, xor a, lane b (or -1), xor b
        plan[..., 2] = -1
        for x in (1, 2, 3):
            m1, i1, _m2, _i2 = small[x]
            a, c = _PAIR[x]
            ma1, ia1, ma2, ia2 = small[a]
            mc1, ic1, mc2, ic2 = small[c]
            clash = ia1 == ic1
            left, right = ma1 + mc2, ma2 + mc1
            pair_cost = np.where(clash, np.minimum(left, right), ma1 + mc1)
            pair_a = np.where(clash & (right < left), ia2, ia1)
            pair_c = np.where(clash & ~(right < left), ic2, ic1)
            single = m1 <= pair_cost
            here = need == x
            repair_cost = np.where(here, np.where(single, m1, pair_cost), repair_cost)
            plan[..., 0] = np.where(here, np.where(single, i1, pair_a), plan[..., 0])
            plan[..., 1] = np.where(here, np.where(single, x, a), plan[..., 1])
            plan[..., 2] = np.where(here, np.where(single, -1, pair_c), plan[..., 2])
            plan[..., 3] = np.where(here, np.where(single, 0, c), plan[..., 3])
        total = total + repair_cost
        state = total.argmin(-1)
        out = np.take_along_axis(sym, state[..., None, None], 2)[:, :, 0, :].copy()
        chosen_plan = np.take_along_axis(plan, state[..., None, None], 2)[:, :, 0, :]          # [R, B, 4]
        need_s = np.take_along_axis(need, state[..., None], 2)[:, :, 0]
        rr, bb = np.nonzero(need_s)
        out[rr, bb, chosen_plan[rr, bb, 0]] ^= chosen_plan[rr, bb, 1]
        two = chosen_plan[rr, bb, 2] >= 0
        out[rr[two], bb[two], chosen_plan[rr[two], bb[two], 2]] ^= chosen_plan[rr[two], bb[two], 3]
    row_err = np.take_along_axis(total, state[..., None], 2)[:, :, 0].sum(1)
    assert np.array_equal(block_tags(out.astype(np.uint8), q), (state & 3).astype(np.uint8))
    return out.astype(np.uint8), (state >> 2).astype(np.uint8), d_of.astype(np.uint8), p_of.astype(np.uint8), row_err


def quantize_mxfp4_sq(src: MxTensor, *, row_q_bits=None, target_bits: float | None = None, matrix_scale_base: int | None = None,
                      importance=None, chunk_bytes: int = 64 << 20) -> Mxfp4SqTensor:
    """``src``: a native MXFP4 matrix.  Give the widths either as ``row_q_bits`` (one value in 1..4 for all rows, or one
    per row) or as ``target_bits``, the mean stored bits per weight to reach (side streams included); ``importance
    [rows]`` weighs the rows' errors in that allocation.  ``q = 4`` rows are copied bit for bit."""
    if src.dtype != MXFP4_DTYPE:
        raise ValueError("MXFP4-SQ re-codes native MXFP4 matrices")
    rows, cols = src.shape
    if cols % 32:
        raise ValueError("MXFP4-SQ needs complete 32-blocks")
    blocks = cols // 32
    packed = np.asarray(src.values, dtype=np.uint8)
    nib = np.empty((rows, cols), dtype=np.uint8)
    nib[:, 0::2], nib[:, 1::2] = packed & 15, packed >> 4
    scales = np.asarray(src.scales, dtype=np.uint8)
    if (row_q_bits is None) == (target_bits is None):
        raise ValueError("give exactly one of row_q_bits and target_bits")
    if row_q_bits is not None:
        q_of = np.broadcast_to(np.asarray(row_q_bits, dtype=np.int64), (rows,)).copy()
        if q_of.min() < 1 or q_of.max() > 4:
            raise ValueError("MXFP4-SQ widths are 1..4")
        widths = sorted(set(q_of.tolist()) - {4})
    else:
        q_of, widths = None, [1, 2, 3]
    compressed = np.ones(rows, dtype=bool) if q_of is None else q_of < 4
    if matrix_scale_base is None:
        base = select_scale_base(nib[compressed], scales[compressed]) if compressed.any() else min(251, int(scales.min()))
    else:
        base = int(matrix_scale_base)
    if not 0 <= base <= 251:
        raise ValueError("the exponent window must leave four valid E8M0 values")
    e_lo, e_hi = min(0, int(scales.min()) - base), max(3, int(scales.max()) - base)
    e_lo, e_hi = max(e_lo, -40), min(e_hi, 40)  # beyond that a block is all-or-nothing anyway; clamping keeps the table finite
    coded = {}
    for q in widths:
        table = _cost_table(q, e_lo, e_hi)
        ids = np.arange(rows) if q_of is None else np.flatnonzero(q_of == q)
        per_row = blocks * 8 * 32 * (1 << q) * 8 * 3
        step = max(1, chunk_bytes // per_row)
        parts = [_encode_rows(nib[ids[i : i + step]].reshape(-1, blocks, 32), scales[ids[i : i + step]], q, base, table, e_lo)
                 for i in range(0, ids.size, step)]
        coded[q] = (ids,) + tuple(np.concatenate([p[j] for p in parts]) for j in range(5))
    if q_of is None:
        q_of = _allocate(rows, cols, {q: coded[q][5] for q in widths}, float(target_bits), importance)
    # assemble in row order
    row_symbols: list[bytes] = [b""] * rows
    sel, ssc, spal, native = [], [], [], []
    where = {q: {int(r): i for i, r in enumerate(coded[q][0])} for q in coded}
    for r in range(rows):
        q = int(q_of[r])
        if q == 4:
            row_symbols[r] = packed[r].tobytes()
            native.append(scales[r])
            continue
        i = where[q][r]
        _ids, sym, selectors, d_of, p_of, _err = coded[q]
        row_symbols[r] = pack_bits(sym[i].reshape(-1), q)
        sel.append(selectors[i])
        ssc.append(d_of[i])
        spal.append(p_of[i])
    stack = lambda items, width: np.stack(items).astype(np.uint8) if items else np.empty((0, width), np.uint8)
    return Mxfp4SqTensor((rows, cols), base, q_of.astype(np.uint8), row_symbols, stack(sel, blocks), stack(ssc, 8), stack(spal, 8),
                         stack(native, blocks))


def _allocate(rows: int, cols: int, errors: dict[int, np.ndarray], target_bits: float, importance) -> np.ndarray:
    """Row widths for a mean of ``target_bits`` stored bits per weight: every row starts lossless and the row whose next
    narrower width adds the least (weighted) error per byte saved is narrowed until the budget is met."""
    weight = np.ones(rows) if importance is None else np.asarray(importance, dtype=np.float64).reshape(rows)
    err = {4: np.zeros(rows), **{q: errors[q] * weight for q in errors}}
    size = {q: row_nbytes(q, cols) for q in (1, 2, 3, 4)}
    q_of = np.full(rows, 4, dtype=np.int64)
    budget = target_bits * cols / 8.0 * rows
    used = float(size[4] * rows)
    heap = [((err[3][r] - err[4][r]) / (size[4] - size[3]), r) for r in range(rows)]
    heapq.heapify(heap)
    while heap and used > budget:
        _price, r = heapq.heappop(heap)
        q = int(q_of[r])
        q_of[r] = q - 1
        used -= size[q] - size[q - 1]
        if q - 1 > 1:
            heapq.heappush(heap, ((err[q - 2][r] - err[q - 1][r]) / (size[q - 1] - size[q - 2]), r))
    return q_of
