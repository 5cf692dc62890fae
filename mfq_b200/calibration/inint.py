"""Per-neuron NINT widths ("inint"): every output row of a dense projection is stored at the narrow or at the wide code
width, chosen by how much error the narrow width costs where it matters.

For each quantizable 2-D weight the matrix is quantized once at each width; a row's loss at a width is its squared
reconstruction error weighted by the input importances (``<name>.in`` of the importance matrix) and by the energy of
the output neuron (``<name>.out``) -- the two halves of the activation-aware objective.  All rows of all tensors then
compete for one budget: with two options per row the multiple-choice knapsack of :mod:`.natscale` reduces to sorting
the rows by loss saved per byte and upgrading until the target bits per weight are spent.  The result is the per-row
width map of the NINTv2 layout (``row_q_bits``), which ``quantize_tensors(row_widths=...)`` / ``mfq quantize
--row-widths`` apply.

Reference: ``mfq/cli.py:650-655`` (``calibrate inint``: per-neuron NINT4 / NINT8 rows), ``mfq/calibration/inint.py``.
"""

from __future__ import annotations

import numpy as np

FORMAT = "mfq.inint-rows.v1"


def _row_losses(w: np.ndarray, bits: int, imp_in, device: str):
    import torch

    from ..formats.nint import dequantize_nint, pack_nint
    from ..quantize.expertwise import parse_profiles
    from ..quantize.nint import quantize_nint
    spec = parse_profiles(f"NINT{bits}")[0].nint
    q = quantize_nint(w, spec, importance=imp_in, device=device)
    err = (np.asarray(dequantize_nint(q), dtype=np.float64).reshape(w.shape) - w) ** 2
    if imp_in is not None:
        err = err * np.asarray(imp_in, dtype=np.float64)[None, :]
    return err.sum(1), len(pack_nint(q)) / w.shape[0]


def select_rows(tensors: dict, target_bpw: float, *, imatrix: dict | None = None, low: int = 4, high: int = 8,
                device: str = "cpu", names=None) -> dict:
    """Choose, for every row of every quantizable 2-D tensor, ``low`` or ``high`` code bits so that the mean storage stays
    within ``target_bpw`` bits per weight.  Returns the ``mfq.inint-rows.v1`` document."""
    from ..quantize import presets
    from .imatrix import input_importance
    if not low < high:
        raise ValueError("low must be narrower than high")
    items = []  # (name, rows, cols, loss_low[rows], loss_high[rows], bytes_low, bytes_high)
    for name in sorted(tensors):
        t = np.asarray(tensors[name])
        if t.ndim != 2 or not presets.quantizable(name, t.shape) or (names is not None and name not in names):
            continue
        w = t.astype(np.float32)
        imp = input_importance(imatrix, name) if imatrix is not None else None
        l_lo, b_lo = _row_losses(w, low, imp, device)
        l_hi, b_hi = _row_losses(w, high, imp, device)
        out_w = np.ones(w.shape[0])
        if imatrix is not None and name + ".out" in imatrix:
            e = np.asarray(imatrix[name + ".out"], dtype=np.float64)
            wn = (w.astype(np.float64) ** 2).sum(1)
            out_w = e / np.maximum(wn, 1e-30)  # per unit of weight energy: how loudly this neuron speaks
            out_w = out_w / max(out_w.mean(), 1e-30)
        items.append((name, w.shape[0], w.shape[1], l_lo * out_w, l_hi * out_w, b_lo, b_hi))
    if not items:
        raise ValueError("no quantizable 2-D tensor to allocate")
    total_weights = sum(r * c for _n, r, c, *_ in items)
    budget = target_bpw * total_weights / 8.0
    base = sum(r * b_lo for _n, r, _c, _ll, _lh, b_lo, _bh in items)
    if base > budget:
        raise ValueError(f"all rows at NINT{low} need {8 * base / total_weights:.3f} bits per weight; the target is {target_bpw}")
    gain = np.concatenate([ll - lh for _n, _r, _c, ll, lh, _bl, _bh in items])
    extra = np.concatenate([np.full(r, bh - bl) for _n, r, _c, _ll, _lh, bl, bh in items])
    order = np.argsort(-(gain / np.maximum(extra, 1e-30)), kind="stable")
    spend = np.cumsum(extra[order])
    take = order[(spend <= budget - base) & (gain[order] > 0)]
    chosen = np.zeros(gain.size, dtype=bool)
    chosen[take] = True
    doc = {"format": FORMAT, "low": low, "high": high, "target_bpw": target_bpw, "tensors": {}}
    off = 0
    used, loss_all_low, loss_now = base, 0.0, 0.0
    for name, r, _c, ll, lh, bl, bh in items:
        sel = chosen[off : off + r]
        doc["tensors"][name] = {"rows": int(r), "high_rows": np.flatnonzero(sel).astype(int).tolist()}
        used += sel.sum() * (bh - bl)
        loss_all_low += float(ll.sum())
        loss_now += float(np.where(sel, lh, ll).sum())
        off += r
    doc["report"] = {"bits_per_weight": 8.0 * used / total_weights, "rows": int(gain.size), "high_rows": int(chosen.sum()),
                     "loss_vs_all_low": loss_now / max(loss_all_low, 1e-30)}
    return doc


def row_bits(doc: dict, name: str):
    """``uint8 [rows]`` code widths of tensor ``name`` from a document of :func:`select_rows` (None if it is not listed)."""
    if doc.get("format") != FORMAT:
        raise ValueError(f"expected {FORMAT}")
    t = doc["tensors"].get(name)
    if t is None:
        return None
    bits = np.full(int(t["rows"]), int(doc["low"]), dtype=np.uint8)
    bits[np.asarray(t["high_rows"], dtype=np.int64)] = int(doc["high"])
    return bits
