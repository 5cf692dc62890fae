"""Numeric experiments on two other ways to spend NVQ2's 15 bits per 8-weight vector (8-bit lattice index + 7 sign
bits): neither has a blob layout or a kernel -- they answer "would it pay" for one tensor, next to the NVQ2 error on the
same tensor.  Scales are NVQ's: an FP16 anchor per row and a 4-bit multiple of it per group of 24 weights.

* additive: ``vector ~ scale * (A[i] + B[j])`` with 256 + 128 signed int8 codewords (8 + 7 index bits); trained by
  alternating assignment (each index re-chosen with the other fixed) and mean updates, the group scales re-solved by
  least squares between rounds;
* product: the vector's halves coded separately, ``concat(A[i], B[j])`` with a 256-entry and a 128-entry table of signed
  4-vectors; two independent k-means problems per round.

Reference: ``mfq/quantize/nvq_additive.py`` and ``nvq_product.py`` (offline experiments there as well).
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import numpy as np
import torch

from ..formats.nvq import NvqSpec
from .nvq import quantize_nvq

__all__ = ["VectorCodeExperiment", "vector_code_experiment"]

GROUP, VEC = 24, 8


@dataclass
class VectorCodeExperiment:
    kind: str
    rel_error: float            # sum (w - rec)^2 / sum w^2
    nvq2_rel_error: float       # plain NVQ2 (256-entry E8 grid) on the same tensor
    bits_per_weight: float      # codes + scales + anchors, tables excluded
    table_bytes: int
    first: np.ndarray           # int8 [256, 8] (additive) or [256, 4] (product)
    second: np.ndarray          # int8 [128, 8] or [128, 4]
    history: list               # rel_error after every round


def _kmeans(points: torch.Tensor, k: int, rounds: int, seed: int) -> torch.Tensor:
    g = torch.Generator().manual_seed(seed)
    n = points.shape[0]
    cent = points[torch.randperm(n, generator=g)[:k]].clone() if n >= k else torch.nn.functional.pad(points, (0, 0, 0, k - n))
    for _ in range(rounds):
        a = torch.cdist(points, cent).argmin(1)
        sums = torch.zeros_like(cent).index_add_(0, a, points)
        cnt = torch.zeros(k).index_add_(0, a, torch.ones(n))
        cent = torch.where(cnt[:, None] > 0, sums / cnt.clamp_min(1)[:, None], cent)
    return cent


def _nearest(points: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    out = torch.empty(points.shape[0], dtype=torch.long)
    for s in range(0, points.shape[0], 65536):
        out[s : s + 65536] = torch.cdist(points[s : s + 65536], table).argmin(1)
    return out


def vector_code_experiment(weight, kind: str = "additive", *, rounds: int = 6, seed: int = 0) -> VectorCodeExperiment:
    """``weight [rows, K]`` with K a multiple of 24.  Runs on the CPU in float32; meant for single matrices."""
    if kind not in ("additive", "product"):
        raise ValueError("kind is 'additive' or 'product'")
    w = torch.as_tensor(np.asarray(weight, dtype=np.float32))
    rows, n = w.shape
    if n % GROUP:
        raise ValueError("the row length must be a multiple of 24")
    ng, nv = n // GROUP, n // VEC
    xg = w.reshape(rows, ng, GROUP)
    # scales as NVQ stores them: anchor * integer in 0..15
    def stored(scale):
        top = scale.amax(1)
        anchor = (top / 15.0).half().float().clamp_min(1e-12)
        sub = torch.round(scale / anchor[:, None]).clamp(0, 15)
        return anchor[:, None] * sub
    scale = stored(xg.abs().amax(-1) / 100.0)                       # codes peak around 100 of 127
    def units(scale):
        return (xg / scale.clamp_min(1e-12)[..., None]).reshape(rows * nv, VEC)
    u = units(scale)
    live = (scale > 0).repeat_interleave(GROUP // VEC, 1).reshape(-1)
    if kind == "additive":
        first = _kmeans(u[live], 256, 8, seed)
        second = _kmeans(u[live] - first[_nearest(u[live], first)], 128, 8, seed + 1)
    else:
        first = _kmeans(u[live][:, :4], 256, 8, seed)
        second = _kmeans(u[live][:, 4:], 128, 8, seed + 1)
    total = float((w * w).sum())
    history = []
    i = j = None
    for _ in range(max(1, rounds)):
        if kind == "additive":
            j = _nearest(u - first[_nearest(u, first)], second) if j is None else j
            i = _nearest(u - second[j], first)
            j = _nearest(u - first[i], second)
            for tab, idx, rest in ((first, i, u - second[j]), (second, j, None)):
                rest = u - first[i] if rest is None else rest
                sums = torch.zeros_like(tab).index_add_(0, idx[live], rest[live])
                cnt = torch.zeros(tab.shape[0]).index_add_(0, idx[live], torch.ones(int(live.sum())))
                tab.copy_(torch.where(cnt[:, None] > 0, sums / cnt.clamp_min(1)[:, None], tab))
            first, second = first.round().clamp(-127, 127), second.round().clamp(-127, 127)
            code = first[i] + second[j]
        else:
            i, j = _nearest(u[:, :4], first), _nearest(u[:, 4:], second)
            for tab, idx, pts in ((first, i, u[:, :4]), (second, j, u[:, 4:])):
                sums = torch.zeros_like(tab).index_add_(0, idx[live], pts[live])
                cnt = torch.zeros(tab.shape[0]).index_add_(0, idx[live], torch.ones(int(live.sum())))
                tab.copy_(torch.where(cnt[:, None] > 0, sums / cnt.clamp_min(1)[:, None], tab))
            first, second = first.round().clamp(-127, 127), second.round().clamp(-127, 127)
            code = torch.cat([first[i], second[j]], 1)
        cg = code.reshape(rows, ng, GROUP)
        num, den = (xg * cg).sum(-1), (cg * cg).sum(-1)
        scale = stored(torch.where(den > 0, num / den.clamp_min(1e-30), scale).clamp_min(0))
        history.append(float(((xg - scale[..., None] * cg) ** 2).sum()) / total)
        u = units(scale)
    base = quantize_nvq(w.numpy(), NvqSpec("e8_256"))
    from ..formats import dequantize
    nvq2 = float(((torch.from_numpy(np.asarray(dequantize(base))) - w) ** 2).sum()) / total
    bits = (15 * rows * nv + 4 * rows * ng + 16 * rows) / float(rows * n)
    return VectorCodeExperiment(kind, history[-1], nvq2, bits, int(first.numel() + second.numel()),
                                first.to(torch.int8).numpy(), second.to(torch.int8).numpy(), history)
