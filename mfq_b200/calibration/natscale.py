"""NatScale: calibration-light precision allocation for routed experts.

Three pieces, each usable alone:

* :func:`natscale_exponent` turns a vector of positive sensitivity scores ``g`` into the exponent ``beta`` for which the
  weights ``g ** (2 beta)`` (normalised) sit exactly ``tau`` nats of Jeffreys divergence away from uniform: the scores'
  dynamic range stops mattering, only their ordering and shape do.  With ``x = log g`` and ``q = softmax(t x)`` the
  equation is ``t (E_q[x] - mean(x)) = tau``, monotone in ``t``, solved by bisection on scores centred at their maximum
  (no power of a raw score is ever formed).
* :func:`allocate_hulls` is the multiple-choice knapsack behind every budgeted choice here: per item the lower convex
  hull of (bytes, loss) over its options, then the hull edges of all items taken in order of loss saved per byte until
  the budget is met; returns the integral choice and the LP lower bound (the first edge that did not fit, taken
  fractionally).
* :func:`expert_candidates` / :func:`allocate` score every routed expert's gate / up / down matrices under a list of
  NINT families (measured relative error, weighted by the importance matrix when one is given), combine them per expert
  as ``w_e * exposure_e * sqrt(P_down,e / H * sum of relative errors)`` over all family triples, and allocate under a
  bits-per-weight target.  Output: the ``mfq.calibration-scheme.v3`` document ``mfq quantize --ew-scheme`` consumes,
  and the ``mfq.ew-candidates.v1`` table ``mfq solve-ew`` consumes.

Reference: ``mfq/calibration/natscale.py:21-66`` (contrast equation), ``:88-150`` (hull allocation), ``:187-334`` (expert
costs and the whole-file allocation); ``mfq/cli.py:639-656`` (``calibrate allocate / candidates``).
"""

from __future__ import annotations

import heapq
import math

import numpy as np

from .ew_solver import CANDIDATES_FORMAT, SCHEME_FORMAT

__all__ = ["natscale_exponent", "realized_contrast", "allocate_hulls", "expert_candidates", "allocate"]


def _logs(scores) -> np.ndarray:
    g = np.asarray(scores, dtype=np.float64).reshape(-1)
    if not np.isfinite(g).all() or (g < 0).any():
        raise ValueError("sensitivity scores must be finite and non-negative")
    x = np.log(g[g > 0])
    if x.size < 2 or np.ptp(x) == 0:
        raise ValueError("sensitivity scores need at least two distinct positive values")
    return x


def _contrast(x: np.ndarray, t: float) -> float:
    z = x - x.max()
    q = np.exp(t * z)
    q /= q.sum()
    return float(t * (q @ z - z.mean()))


def realized_contrast(scores, beta: float) -> float:
    """Jeffreys divergence (nats) between ``softmax(2 beta log g)`` and the uniform distribution."""
    return _contrast(_logs(scores), 2.0 * beta)


def natscale_exponent(scores, tau: float = 1.0) -> float:
    if not (math.isfinite(tau) and tau > 0):
        raise ValueError("tau must be positive")
    x = _logs(scores)
    span = float(np.ptp(x))
    z = (x - x.max()) / span  # in [-1, 0]: the bisection variable is t * span
    lo, hi = 0.0, 1.0
    while _contrast(z, hi) < tau:
        hi *= 2.0
        if hi > 1e12:
            raise ValueError("the requested contrast cannot be reached")
    for _ in range(200):
        mid = 0.5 * (lo + hi)
        if _contrast(z, mid) < tau:
            lo = mid
        else:
            hi = mid
    return 0.5 * (lo + hi) / (2.0 * span)


def _lower_hull(sizes: np.ndarray, losses: np.ndarray) -> list[int]:
    """Indices of the options on the lower convex hull of (size, loss), by increasing size and decreasing loss."""
    order = sorted(range(len(sizes)), key=lambda i: (sizes[i], losses[i], i))
    hull: list[int] = []
    for i in order:
        if hull and sizes[i] == sizes[hull[-1]]:
            continue  # same size, not better
        if hull and losses[i] >= losses[hull[-1]]:
            continue  # larger and no better
        while len(hull) >= 2:
            a, b = hull[-2], hull[-1]
            if (losses[b] - losses[a]) * (sizes[i] - sizes[b]) <= (losses[i] - losses[b]) * (sizes[b] - sizes[a]):
                break  # slope a->b is steeper (more negative) than b->i: b stays
            hull.pop()
        hull.append(i)
    return hull


def allocate_hulls(payload, costs, budget: int) -> dict:
    """``payload [items, options]`` (or ``[options]``) bytes, ``costs [items, options]`` losses, ``budget`` bytes.
    Returns ``{"choice", "bytes", "objective", "lower_bound"}``; raises if even the smallest options do not fit."""
    costs = np.asarray(costs, dtype=np.float64)
    if costs.ndim != 2 or not np.isfinite(costs).all() or (costs < 0).any():
        raise ValueError("costs must be a finite non-negative [items, options] matrix")
    sizes = np.broadcast_to(np.asarray(payload, dtype=np.int64), costs.shape)
    choice = np.zeros(costs.shape[0], dtype=np.int64)
    heap, used, objective = [], 0, 0.0
    hulls = []
    for r in range(costs.shape[0]):
        h = _lower_hull(sizes[r], costs[r])
        hulls.append(h)
        choice[r] = h[0]
        used += int(sizes[r, h[0]])
        objective += float(costs[r, h[0]])
        if len(h) > 1:
            extra, gain = int(sizes[r, h[1]] - sizes[r, h[0]]), float(costs[r, h[0]] - costs[r, h[1]])
            heapq.heappush(heap, (-gain / extra, r, 0))
    if used > budget:
        raise ValueError(f"the smallest options need {used} bytes, the budget is {budget}")
    lower, fractional = objective, False
    while heap:
        _slope, r, pos = heapq.heappop(heap)
        h = hulls[r]
        extra, gain = int(sizes[r, h[pos + 1]] - sizes[r, h[pos]]), float(costs[r, h[pos]] - costs[r, h[pos + 1]])
        if not fractional:
            if used + extra > budget:
                lower -= (budget - used) / extra * gain
                fractional = True
            else:
                lower -= gain
        if choice[r] == h[pos] and used + extra <= budget:  # an item stops at its first edge that does not fit
            choice[r] = h[pos + 1]
            used += extra
            objective -= gain
            if pos + 2 < len(h):
                e2, g2 = int(sizes[r, h[pos + 2]] - sizes[r, h[pos + 1]]), float(costs[r, h[pos + 1]] - costs[r, h[pos + 2]])
                heapq.heappush(heap, (-g2 / e2, r, pos + 1))
    return {"choice": choice, "bytes": int(used), "objective": float(objective), "lower_bound": float(max(0.0, lower))}


def _family_spec(family: str):
    from ..quantize.expertwise import parse_profiles
    prof = parse_profiles(family)[0]
    if prof.nint is None:
        raise ValueError(f"{family}: only NINT families are scored here")
    return prof.nint


def expert_candidates(tensors: dict, families: list[str], imatrix: dict | None = None, layers: set[int] | None = None) -> dict:
    """Quantize every routed expert matrix under every family and record relative error and packed size.
    ``tensors``: canonical name -> array; expert banks are ``[experts, out, in]``.  Returns the ``mfq.ew-candidates.v1``
    document (one entry per bank, per expert a candidate per family)."""
    import torch

    from ..formats.nint import dequantize_nint, pack_nint
    from ..quantize.nint import quantize_nint
    specs = {f: _family_spec(f) for f in families}
    out = []
    for name in sorted(tensors):
        t = np.asarray(tensors[name])
        if ".mlp.experts." not in name or t.ndim != 3:
            continue
        layer = int(name.split(".")[2])
        if layers is not None and layer not in layers:
            continue
        projection = name.split(".")[-2]
        experts = []
        for e in range(t.shape[0]):
            w = torch.from_numpy(np.ascontiguousarray(t[e], dtype=np.float32))
            imp = None
            if imatrix is not None and f"{name}#{e}.in" in imatrix:
                v = np.asarray(imatrix[f"{name}#{e}.in"], dtype=np.float64)
                imp = torch.from_numpy((v / max(v.mean(), 1e-30)).clip(1e-6).astype(np.float32))
            energy = float(((w.double() ** 2) * (imp.double()[None, :] if imp is not None else 1.0)).sum()) + 1e-30
            cands = []
            for fam, spec in specs.items():
                q = quantize_nint(w, spec, importance=imp)
                rec = torch.from_numpy(np.asarray(dequantize_nint(q), dtype=np.float32)).reshape(w.shape)
                nbits = 8 * len(pack_nint(q))
                err = ((rec - w).double() ** 2) * (imp.double()[None, :] if imp is not None else 1.0)
                cands.append({"family": fam, "distortion": float(err.sum() / energy),
                              "variable_storage_bits": nbits, "effective_bpw": nbits / w.numel()})
            experts.append({"expert_id": e, "weights": int(w.numel()), "candidates": cands})
        out.append({"name": name, "layer": layer, "projection": projection, "fixed_storage_bits": 0, "experts": experts})
    return {"format": CANDIDATES_FORMAT, "families": list(families), "tensors": out}


def allocate(candidates: dict, target_bpw: float, *, imatrix: dict | None = None, tensors: dict | None = None, tau: float = 1.0,
             sensitivity: str = "imatrix-energy") -> tuple[dict, dict]:
    """Joint gate / up / down family per routed expert under ``target_bpw`` mean bits per expert weight.

    ``sensitivity``: ``uniform`` (all experts weigh the same), ``imatrix-energy`` (weights ``P_down ** beta`` with the
    NatScale exponent; needs ``imatrix`` and ``tensors``) or ``reap`` (the expert's router-weighted activation norm,
    ``<down>#e.reap`` of an importance matrix collected with expert saliencies, in place of the output energy).  Exposure is the fraction of calibration rows an expert saw
    (1 without an importance matrix).  Returns ``(scheme, report)``."""
    if candidates.get("format") != CANDIDATES_FORMAT:
        raise ValueError(f"expected {CANDIDATES_FORMAT}")
    by_layer: dict[int, dict[str, dict]] = {}
    for t in candidates["tensors"]:
        by_layer.setdefault(int(t["layer"]), {})[t["projection"]] = t
    rows_cost, rows_bytes, index = [], [], []
    scores, exposure = [], []
    total_weights = 0
    for layer, banks in sorted(by_layer.items()):
        if set(banks) != {"gate", "up", "down"}:
            raise ValueError(f"layer {layer}: gate, up and down banks are all needed")
        fams = [c["family"] for c in banks["gate"]["experts"][0]["candidates"]]
        q = len(fams)
        combos = np.stack(np.meshgrid(np.arange(q), np.arange(q), np.arange(q), indexing="ij"), -1).reshape(-1, 3)
        n_experts = len(banks["gate"]["experts"])
        counts = np.ones(n_experts)
        if imatrix is not None:
            counts = np.array([float(imatrix.get(f"{banks['gate']['name']}#{e}.count", 0)) for e in range(n_experts)])
        denom = max(counts.max(), 1.0)
        for e in range(n_experts):
            rel = np.zeros((3, q))
            byt = np.zeros((3, q), dtype=np.int64)
            for pi, proj in enumerate(("gate", "up", "down")):
                ex = banks[proj]["experts"][e]
                if [c["family"] for c in ex["candidates"]] != fams:
                    raise ValueError("every expert must list the same families in the same order")
                rel[pi] = [c["distortion"] for c in ex["candidates"]]
                byt[pi] = [int(math.ceil(c["variable_storage_bits"] / 8)) for c in ex["candidates"]]
                total_weights += int(ex["weights"])
            p_down = 1.0
            if sensitivity == "imatrix-energy":
                if imatrix is None or tensors is None:
                    raise ValueError("imatrix-energy sensitivity needs the importance matrix and the weights")
                w = np.asarray(tensors[banks["down"]["name"]][e], dtype=np.float64)
                second = np.asarray(imatrix.get(f"{banks['down']['name']}#{e}.in", np.zeros(w.shape[1])), dtype=np.float64)
                p_down = float((second[None, :] * w * w).sum()) / w.shape[0]  # output energy of the down projection per channel
            elif sensitivity == "reap":
                if imatrix is None:
                    raise ValueError("reap sensitivity needs an importance matrix collected with expert saliencies")
                reap = float(np.asarray(imatrix.get(f"{banks['down']['name']}#{e}.reap", 0.0)))
                p_down = reap * reap  # the loss below takes the square root: an expert weighs by its saliency itself
            f = counts[e] / denom
            loss = f * np.sqrt(p_down * (rel[0, combos[:, 0]] + rel[1, combos[:, 1]] + rel[2, combos[:, 2]]))
            rows_cost.append(loss)
            rows_bytes.append(byt[0, combos[:, 0]] + byt[1, combos[:, 1]] + byt[2, combos[:, 2]])
            index.append((layer, e, fams, combos))
            scores.append(p_down)
            exposure.append(f)
    costs = np.stack(rows_cost)
    beta, contrast = 0.0, 0.0
    if sensitivity in ("imatrix-energy", "reap"):
        g = np.asarray(scores)
        beta = natscale_exponent(g, tau)
        contrast = realized_contrast(g, beta)
        wts = np.zeros_like(g)
        pos = g > 0
        lg = np.log(g[pos])
        wts[pos] = np.exp(beta * (lg - lg.max()))
        costs = costs * wts[:, None]
    elif sensitivity != "uniform":
        raise ValueError("sensitivity must be uniform, imatrix-energy or reap")
    budget = int(target_bpw * total_weights / 8)
    sol = allocate_hulls(np.stack(rows_bytes), costs, budget)
    assignments, hist = [], {}
    for (layer, e, fams, combos), ci in zip(index, sol["choice"]):
        for pi, proj in enumerate(("gate", "up", "down")):
            fam = fams[int(combos[ci, pi])]
            bank = by_layer[layer][proj]
            cand = bank["experts"][e]["candidates"][int(combos[ci, pi])]
            assignments.append({"tensor": bank["name"], "layer": layer, "projection": proj, "expert_id": e, "family": fam,
                                "effective_bpw": cand.get("effective_bpw")})
            hist[fam] = hist.get(fam, 0) + 1
    scheme = {"format": SCHEME_FORMAT, "kind": "expert-wise", "method": "NatScale", "assignments": assignments}
    report = {"method": "NatScale", "sensitivity": sensitivity, "tau": tau, "beta": beta, "realized_contrast": contrast,
              "objective": sol["objective"], "lower_bound": sol["lower_bound"],
              "relative_gap": (sol["objective"] - sol["lower_bound"]) / sol["objective"] if sol["objective"] else 0.0,
              "bits_per_weight": 8.0 * sol["bytes"] / max(1, total_weights), "target_bpw": target_bpw,
              "family_histogram": dict(sorted(hist.items())),
              "exposure": {"min": float(min(exposure)), "max": float(max(exposure)), "zero": int(sum(1 for f in exposure if f == 0))},
              "formula": "w * exposure * sqrt(P_down / H * sum of relative errors)"}
    return scheme, report
