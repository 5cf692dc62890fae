"""Expert-wise joint budget solver: importance table + rate/distortion candidates + budget -> calibration scheme.

Inputs follow the reference's documents (``docs/quantization/ew-joint-solver.md``): ``mfq.ew-importance.v1`` (score or
rank mode, optional normalisation), ``mfq.ew-candidates.v1`` (per tensor: ``fixed_storage_bits`` and, per expert, a
list of candidates with ``distortion``, ``effective_bpw``, ``variable_storage_bits`` and an optional ``pool_key`` whose
``pool_storage_bits`` is paid once when any expert of the tensor uses the pool).  The allocation is a 0/1 program

    min  sum_{t,e,c} w[t,e] * distortion[t,e,c] * x[t,e,c]
    s.t. sum_c x[t,e,c] = 1;   x[t,e,c] <= y[t,pool(c)];   fixed + sum variable*x + sum pool*y <= budget

solved with ``scipy.optimize.milp`` (HiGHS).  Output: ``mfq.calibration-scheme.v3`` (one family per expert projection)
plus a report.  Reference: ``mfq/calibration/ew_solver.py``.
"""

from __future__ import annotations

import json
from pathlib import Path

import numpy as np

IMPORTANCE_FORMAT = "mfq.ew-importance.v1"
CANDIDATES_FORMAT = "mfq.ew-candidates.v1"
SCHEME_FORMAT = "mfq.calibration-scheme.v3"
_PROJECTIONS = ("gate", "up", "down")


def _rank_weight(rank: int, n: int, policy: str) -> float:
    if policy == "linear_percentile":
        return (n - rank + 1) / n
    if policy == "reciprocal":
        return 1.0 / rank
    if policy == "uniform":
        return 1.0
    raise ValueError(f"unknown rank_weighting {policy!r}")


def importance_weights(doc: dict) -> dict[tuple[int, int, str], float]:
    """``{(layer, expert, projection): weight}``; an entry without ``projection`` covers gate, up and down, an
    entry with one overrides it."""
    if doc.get("format") != IMPORTANCE_FORMAT:
        raise ValueError(f"expected {IMPORTANCE_FORMAT}")
    mode = doc.get("mode", "score")
    shared, exact = {}, {}
    entries = doc["entries"]
    if mode == "rank":
        policy = doc.get("rank_weighting", "linear_percentile")
        by_layer: dict[int, list] = {}
        for e in entries:
            by_layer.setdefault(int(e["layer"]), []).append(e)
        for layer, es in by_layer.items():
            ranks = sorted(int(e["rank"]) for e in es)
            if ranks != list(range(1, len(es) + 1)):
                raise ValueError(f"layer {layer}: ranks must be unique and contiguous 1..N")
            for e in es:
                shared[(layer, int(e["expert_id"]))] = _rank_weight(int(e["rank"]), len(es), policy)
    else:
        for e in entries:
            key = (int(e["layer"]), int(e["expert_id"]))
            if "projection" in e:
                exact[key + (e["projection"],)] = float(e["score"])
            else:
                shared[key] = float(e["score"])
    out = {}
    for (layer, expert), s in shared.items():
        for p in _PROJECTIONS:
            out[(layer, expert, p)] = s
    out.update(exact)
    norm = doc.get("score_normalization", "none")
    if norm != "none":
        def group(k):
            return {"global_sum": 0, "layer_sum": k[0], "layer_projection_sum": (k[0], k[2]), "tensor_sum": (k[0], k[2])}[norm]
        totals: dict = {}
        for k, v in out.items():
            totals[group(k)] = totals.get(group(k), 0.0) + v
        out = {k: v / max(totals[group(k)], 1e-30) for k, v in out.items()}
    return out


def solve(importance: dict, candidates: dict, budget_bits: float, time_limit: float = 60.0) -> tuple[dict, dict]:
    """Returns ``(scheme, report)``."""
    from scipy.optimize import Bounds, LinearConstraint, milp
    from scipy.sparse import lil_matrix

    if candidates.get("format") != CANDIDATES_FORMAT:
        raise ValueError(f"expected {CANDIDATES_FORMAT}")
    w = importance_weights(importance)
    xs, ys = [], {}  # x: (tensor, expert, candidate dict); y: (tensor, pool_key) -> index
    fixed = 0.0
    for t in candidates["tensors"]:
        fixed += float(t.get("fixed_storage_bits", 0))
        for ex in t["experts"]:
            for c in ex["candidates"]:
                xs.append((t, ex, c))
                if c.get("pool_key") is not None:
                    ys.setdefault((t["name"], c["pool_key"]), (len(ys), float(c.get("pool_storage_bits", 0))))
    nx, ny = len(xs), len(ys)
    cost = np.zeros(nx + ny)
    storage = np.zeros(nx + ny)
    for i, (t, ex, c) in enumerate(xs):
        weight = w.get((int(t["layer"]), int(ex["expert_id"]), t["projection"]), 1.0)
        cost[i] = weight * float(c["distortion"])
        storage[i] = float(c.get("variable_storage_bits", 0))
    for (idx, bits) in ys.values():
        storage[nx + idx] = bits
    groups: dict = {}
    for i, (t, ex, _c) in enumerate(xs):
        groups.setdefault((t["name"], int(ex["expert_id"])), []).append(i)
    rows = len(groups) + sum(1 for _t, _e, c in xs if c.get("pool_key") is not None) + 1
    a = lil_matrix((rows, nx + ny))
    lb, ub = np.zeros(rows), np.zeros(rows)
    r = 0
    for idxs in groups.values():
        for i in idxs:
            a[r, i] = 1
        lb[r] = ub[r] = 1
        r += 1
    for i, (t, _ex, c) in enumerate(xs):
        if c.get("pool_key") is not None:
            a[r, i] = 1
            a[r, nx + ys[(t["name"], c["pool_key"])][0]] = -1
            lb[r], ub[r] = -np.inf, 0
            r += 1
    a[r, :] = storage
    lb[r], ub[r] = -np.inf, budget_bits - fixed
    res = milp(cost, constraints=LinearConstraint(a.tocsr(), lb, ub), integrality=np.ones(nx + ny), bounds=Bounds(0, 1),
               options={"time_limit": time_limit})
    if res.x is None:
        raise ValueError(f"no allocation fits the budget ({res.message})")
    chosen = [xs[i] for i in range(nx) if res.x[i] > 0.5]
    assignments = [{"tensor": t["name"], "layer": int(t["layer"]), "projection": t["projection"], "expert_id": int(ex["expert_id"]),
                    "family": c["family"], "effective_bpw": c.get("effective_bpw")} for t, ex, c in chosen]
    used = fixed + float(storage @ np.round(res.x))
    scheme = {"format": SCHEME_FORMAT, "kind": "expert-wise", "assignments": assignments}
    report = {"objective": float(res.fun), "storage_bits": used, "budget_bits": float(budget_bits), "status": res.message,
              "family_histogram": {f: sum(a_["family"] == f for a_ in assignments) for f in sorted({a_["family"] for a_ in assignments})}}
    return scheme, report


def solve_files(importance_path, candidates_path, budget_path, scheme_out, report_out=None) -> dict:
    imp, cand, budget = (json.loads(Path(p).read_text()) for p in (importance_path, candidates_path, budget_path))
    scheme, report = solve(imp, cand, float(budget["budget_bits"]))
    Path(scheme_out).write_text(json.dumps(scheme, indent=1))
    if report_out:
        Path(report_out).write_text(json.dumps(report, indent=1))
    return report
