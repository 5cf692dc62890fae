"""AlphaQ: calibration-free importance of weight matrices from their spectra, and budgeted width allocation.

For a matrix ``W``: cut it into complete 128x128 blocks, pool the squared singular values, estimate the tail index
with the Hill estimator over the top ``k = min(n-1, max(10, floor(0.1 n)))`` eigenvalues,
``alpha = 1 + k / sum(log(tail / threshold))``; importance ``I = median(alpha) / alpha * Var(W)`` (heavy-tailed,
high-variance matrices are important).  Allocation minimises ``sum_i I_i * 2^(-2 b_i)`` under a size budget.
Method as documented in ``docs/quantization/alphaq.md:10-32`` of the reference (``mfq/calibration/alphaq.py``); the
allocation here is an exact multiple-choice knapsack by Lagrangian bisection with a greedy repair step.
"""

from __future__ import annotations

from dataclasses import dataclass

import numpy as np

BLOCK = 128
_FLOOR = 1e-12


def pooled_spectrum(w: np.ndarray) -> np.ndarray:
    """Squared singular values of all complete 128x128 blocks (of the whole matrix when a side is < 128)."""
    w = np.asarray(w, dtype=np.float32)
    r, c = w.shape
    if r < BLOCK or c < BLOCK:
        return np.linalg.svd(w, compute_uv=False).astype(np.float64) ** 2
    br, bc = r // BLOCK, c // BLOCK
    blocks = w[: br * BLOCK, : bc * BLOCK].reshape(br, BLOCK, bc, BLOCK).transpose(0, 2, 1, 3).reshape(-1, BLOCK, BLOCK)
    return (np.linalg.svd(blocks, compute_uv=False).astype(np.float64) ** 2).reshape(-1)


def hill_alpha(eigs: np.ndarray) -> float:
    lam = np.sort(np.maximum(np.asarray(eigs, dtype=np.float64), _FLOOR))
    n = lam.size
    if n < 2:
        return 1.0
    k = min(n - 1, max(10, int(0.1 * n)))
    thr = lam[n - k - 1]
    s = np.log(np.maximum(lam[n - k :], _FLOOR) / max(thr, _FLOOR)).sum()
    return float(1.0 + k / max(s, _FLOOR))


@dataclass
class WeightStats:
    alpha: float
    variance: float
    size: int


def weight_statistics(w: np.ndarray) -> WeightStats:
    w = np.asarray(w, dtype=np.float32)
    var = float(w.astype(np.float64).var())
    if var == 0.0:
        return WeightStats(1.0, 0.0, w.size)
    return WeightStats(hill_alpha(pooled_spectrum(w.reshape(w.shape[0], -1))), var, w.size)


def importance(stats: dict[str, WeightStats]) -> dict[str, float]:
    """``I = median(alpha) / alpha * Var`` with one global positive scale for numerical comfort."""
    med = float(np.median([s.alpha for s in stats.values()]))
    raw = {k: (med / s.alpha) * s.variance for k, s in stats.items()}
    scale = max(raw.values()) or 1.0
    return {k: v / scale for k, v in raw.items()}


def allocate(imp: dict[str, float], sizes: dict[str, int], candidates: dict[str, float], budget_bits: float) -> dict[str, str]:
    """Pick one candidate (name -> bits per weight used for BOTH scoring and storage) per tensor, minimising
    ``sum I * 2^(-2 b)`` with ``sum size * b <= budget_bits``.  Returns ``{tensor: candidate}``."""
    names = sorted(candidates, key=candidates.get)
    bits = np.array([candidates[n] for n in names])
    keys = list(imp)
    cost = np.array([[imp[k] * 2.0 ** (-2.0 * b) for b in bits] for k in keys])
    size = np.array([[sizes[k] * b for b in bits] for k in keys])
    if size[:, 0].sum() > budget_bits:
        raise ValueError("budget below the smallest candidate for every tensor")

    def pick(lmbda):
        return np.argmin(cost + lmbda * size, axis=1)

    lo, hi = 0.0, 1.0
    while size[np.arange(len(keys)), pick(hi)].sum() > budget_bits:
        hi *= 4.0
    for _ in range(80):
        mid = 0.5 * (lo + hi)
        if size[np.arange(len(keys)), pick(mid)].sum() > budget_bits:
            lo = mid
        else:
            hi = mid
    choice = pick(hi)
    # greedy repair: spend what the bisection left over on the best marginal upgrades
    used = size[np.arange(len(keys)), choice].sum()
    while True:
        best, gain = None, 0.0
        for i, c in enumerate(choice):
            if c + 1 < len(bits):
                extra = size[i, c + 1] - size[i, c]
                if used + extra <= budget_bits:
                    g = (cost[i, c] - cost[i, c + 1]) / max(extra, 1e-30)
                    if g > gain:
                        best, gain = i, g
        if best is None:
            break
        used += size[best, choice[best] + 1] - size[best, choice[best]]
        choice[best] += 1
    return {k: names[c] for k, c in zip(keys, choice)}
