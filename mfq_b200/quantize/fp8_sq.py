"""FP8-SQ palette quantizer: shrink an E4M3 matrix below 8 bits per weight without leaving the E4M3 value set.

An ``FP8-128SQ`` / ``MXFP8-SQ`` tensor stores each row either raw (SQ8) or as ``q``-bit symbols into one matrix-wide
palette of ``2**q`` legal E4M3 codes (``formats/fp8sq.py``).  This module fits those palettes and picks every row's
width:

* :func:`fit_palette`: the weighted one-dimensional clustering of the matrix's E4M3 levels into ``2**q`` clusters is
  solved exactly by dynamic programming over the (at most 254) occupied levels in value order; a cluster's
  representative is the occupied level nearest its weighted mean, so every palette entry is a code the source already
  uses and the reconstruction stays native E4M3;
* :func:`quantize_fp8_sq`: fits the seven palettes, evaluates every row's weighted error at every width and lowers
  row widths greedily -- always the step with the least error added per bit saved -- until the requested mean width is
  met.

Reference: ``mfq/quantize/fp8_sq.py:137-235`` (exact palette DP), ``:379-460`` (row-width allocation).
"""

from __future__ import annotations

import heapq

import numpy as np

from ..formats.fp8sq import Fp8SqTensor, palette_slice
from ..formats.mx import E4M3_TABLE

__all__ = ["fit_palette", "quantize_fp8_sq"]

# finite E4M3 codes in value order (negative zero folded into zero)
_CODES = np.array(sorted((c for c in range(256) if (c & 0x7F) != 0x7F and c != 0x80), key=lambda c: float(E4M3_TABLE[c])), dtype=np.uint8)
_VALUES = E4M3_TABLE[_CODES].astype(np.float64)
_LEVEL_OF = np.zeros(256, dtype=np.int16)
_LEVEL_OF[_CODES] = np.arange(_CODES.size)
_LEVEL_OF[0x80] = _LEVEL_OF[0x00]


def _segment_cost(values: np.ndarray, weights: np.ndarray):
    """``cost[i, j]`` / ``rep[i, j]``: weighted squared error and best representative (an index into ``values``) when
    levels ``i..j`` form one cluster."""
    n = values.size
    pw = np.concatenate([[0.0], np.cumsum(weights)])
    px = np.concatenate([[0.0], np.cumsum(weights * values)])
    px2 = np.concatenate([[0.0], np.cumsum(weights * values * values)])
    cost = np.full((n, n), np.inf)
    rep = np.zeros((n, n), dtype=np.int32)
    ends = np.arange(n)
    for i in range(n):
        j = ends[i:]
        tw, tx, tx2 = pw[j + 1] - pw[i], px[j + 1] - px[i], px2[j + 1] - px2[i]
        mean = tx / np.maximum(tw, 1e-300)
        pos = np.clip(np.searchsorted(values, mean), i, j)  # nearest occupied level to the mean, inside the segment
        left = np.maximum(pos - 1, i)
        pick = np.where(np.abs(values[left] - mean) <= np.abs(values[pos] - mean), left, pos)
        r = values[pick]
        cost[i, i:] = tx2 - 2.0 * r * tx + r * r * tw
        rep[i, i:] = pick
    return cost, rep


def fit_palette(codes: np.ndarray, weights: np.ndarray | None, bits: int) -> np.ndarray:
    """``2**bits`` distinct E4M3 codes minimizing the weighted squared error of mapping every element of ``codes`` to its
    nearest palette entry (exact).  Unused slots are filled with further legal codes so the palette stays duplicate-free."""
    if not 1 <= bits <= 7:
        raise ValueError("palettes exist for SQ1..SQ7")
    lv = _LEVEL_OF[np.asarray(codes, dtype=np.uint8)].reshape(-1)
    w = np.ones(lv.size) if weights is None else np.asarray(weights, dtype=np.float64).reshape(-1)
    hist = np.bincount(lv, weights=w, minlength=_CODES.size)
    active = np.flatnonzero(hist > 0)
    k = 1 << bits
    if active.size <= k:
        chosen = list(active)
    else:
        values, wts = _VALUES[active], hist[active]
        cost, rep = _segment_cost(values, wts)
        n = active.size
        best = np.full(n + 1, np.inf)
        best[0] = 0.0
        back = np.zeros((k + 1, n + 1), dtype=np.int32)
        for g in range(1, k + 1):
            cur = np.full(n + 1, np.inf)
            for end in range(g, n + 1):
                begins = np.arange(g - 1, end)
                cand = best[begins] + cost[begins, end - 1]
                j = int(np.argmin(cand))
                cur[end], back[g, end] = cand[j], begins[j]
            best = cur
        chosen, end = [], n
        for g in range(k, 0, -1):
            begin = int(back[g, end])
            chosen.append(int(active[rep[begin, end - 1]]))
            end = begin
        chosen.reverse()
    have = set(int(c) for c in chosen)
    spare = (i for i in range(_CODES.size) if i not in have)
    while len(chosen) < k:
        chosen.append(next(spare))
    return _CODES[np.sort(np.asarray(chosen))]


def _snap(codes: np.ndarray, palette: np.ndarray) -> np.ndarray:
    """Every code replaced by the palette entry nearest in value."""
    pv = E4M3_TABLE[palette].astype(np.float64)
    order = np.argsort(pv)
    pv, pal = pv[order], palette[order]
    x = E4M3_TABLE[codes].astype(np.float64)
    pos = np.clip(np.searchsorted(pv, x), 1, pv.size - 1)
    left = pos - 1
    pick = np.where(np.abs(pv[left] - x) <= np.abs(pv[pos] - x), left, pos)
    return pal[pick]


def quantize_fp8_sq(t: Fp8SqTensor, target_bits: float, importance: np.ndarray | None = None) -> Fp8SqTensor:
    """Re-encode an E4M3 tensor (raw rows) with per-row palette widths averaging ``target_bits`` code bits per weight.
    ``importance``: optional non-negative weight per input column.  Scales and block geometry are kept."""
    if not 1.0 <= target_bits <= 8.0:
        raise ValueError("target_bits must lie in [1, 8]")
    codes = np.asarray(t.codes, dtype=np.uint8)
    rows, cols = codes.shape
    w = np.ones((rows, cols)) if importance is None else np.broadcast_to(np.asarray(importance, dtype=np.float64)[None, :], codes.shape)
    # an element's error in real units carries its block multiplier (squared)
    if t.scale_dtype != "F8_E8M0":
        br, bc = t.block_shape
        mult = np.repeat(np.repeat(np.asarray(t.scales, dtype=np.float64), br, 0)[:rows], bc, 1)[:, :cols]
        w = w * mult * mult
    x = E4M3_TABLE[codes].astype(np.float64)
    palettes = np.asarray(t.palettes, dtype=np.uint8).copy()
    snapped, err = {}, np.zeros((9, rows))
    for q in range(1, 8):
        pal = fit_palette(codes, w, q)
        palettes[palette_slice(q)] = pal
        snapped[q] = _snap(codes, pal)
        d = E4M3_TABLE[snapped[q]].astype(np.float64) - x
        err[q] = (w * d * d).sum(1)
    widths = np.full(rows, 8, dtype=np.int64)
    budget = rows * (8.0 - target_bits)  # bits per weight to remove, summed over rows
    heap = [((err[7, r] - err[8, r]), r) for r in range(rows)]
    heapq.heapify(heap)
    saved = 0.0
    while heap and saved + 1e-9 < budget:
        _cost, r = heapq.heappop(heap)
        widths[r] -= 1
        saved += 1.0
        if widths[r] > 1:
            heapq.heappush(heap, (err[widths[r] - 1, r] - err[widths[r], r], r))
    out = codes.copy()
    for q in range(1, 8):
        sel = widths == q
        if sel.any():
            out[sel] = snapped[q][sel]
    return Fp8SqTensor(t.dtype, t.shape, out, t.scales, t.block_shape, t.scale_dtype, widths.astype(np.uint8), palettes)
