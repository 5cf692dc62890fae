"""Importance matrices: per-linear-layer input-channel energy (and output-neuron energy) gathered on calibration
text, used as the per-coordinate weights of the NINT least-squares search (``quantize_nint(importance=...)``).

Collection hooks the inputs of the reference fp32 model (``mfq_b200.models.moe_lm.MoeLM`` or any module tree whose
linear weights carry canonical names); statistics are running means of ``x^2`` (inputs) and ``y^2`` (outputs), the
"NAQ" pair of the reference (``mfq/calibration/imatrix.py``).  Stored as ``.npz`` with ``<name>.in`` / ``<name>.out``.
"""

from __future__ import annotations

from pathlib import Path

import numpy as np
import torch


class ImatrixCollector:
    def __init__(self) -> None:
        self.sum_in: dict[str, torch.Tensor] = {}
        self.sum_out: dict[str, torch.Tensor] = {}
        self.count: dict[str, int] = {}
        self.sum_reap: dict[str, float] = {}
        self.n_reap: dict[str, int] = {}

    def observe(self, name: str, x: torch.Tensor, y: torch.Tensor | None = None) -> None:
        """``x [tokens, in]`` the input of linear ``name`` (``y [tokens, out]`` its output, optional)."""
        x = x.detach().reshape(-1, x.shape[-1]).float()
        s = (x * x).sum(0)
        self.sum_in[name] = self.sum_in.get(name, 0) + s
        self.count[name] = self.count.get(name, 0) + x.shape[0]
        if y is not None:
            y = y.detach().reshape(-1, y.shape[-1]).float()
            self.sum_out[name] = self.sum_out.get(name, 0) + (y * y).sum(0)

    def observe_reap(self, name: str, route_weight: torch.Tensor, y: torch.Tensor) -> None:
        """Router-weighted activation norm of one expert (``name`` = ``<down tensor>#<expert>``): ``route_weight [n]`` of
        the tokens routed to it and its outputs ``y [n, hidden]`` before the weighting.  The mean of ``weight * |y|`` over
        the expert's tokens is its REAP saliency: how much it moves the residual stream when it is called."""
        y = y.detach().reshape(-1, y.shape[-1]).float()
        s = float((route_weight.detach().reshape(-1).float() * y.norm(dim=-1)).sum())
        self.sum_reap[name] = self.sum_reap.get(name, 0.0) + s
        self.n_reap[name] = self.n_reap.get(name, 0) + y.shape[0]

    def hook_linear(self, weights: dict[str, torch.Tensor]):
        """Returns ``linear(name, x)`` that multiplies by ``weights[name]`` and records the statistics."""
        def linear(name: str, x: torch.Tensor) -> torch.Tensor:
            y = x @ weights[name].T
            self.observe(name, x, y)
            return y
        return linear

    def result(self) -> dict[str, np.ndarray]:
        out = {}
        for name, s in self.sum_in.items():
            n = max(1, self.count[name])
            out[name + ".in"] = (s / n).cpu().numpy().astype(np.float32)
            out[name + ".count"] = np.array(self.count[name], dtype=np.int64)  # rows seen: an expert's exposure
            if name in self.sum_out:
                out[name + ".out"] = (self.sum_out[name] / n).cpu().numpy().astype(np.float32)
        for name, s in self.sum_reap.items():
            out[name + ".reap"] = np.array(s / max(1, self.n_reap[name]), dtype=np.float64)
        return out

    def save(self, path) -> None:
        np.savez(Path(path), **self.result())


def load(path) -> dict[str, np.ndarray]:
    with np.load(Path(path)) as z:
        return {k: z[k] for k in z.files}


def input_importance(imatrix: dict[str, np.ndarray], name: str, floor: float = 1e-6) -> np.ndarray | None:
    """Per-input-coordinate weights for ``quantize_nint`` (mean-normalised, floored), or None if not collected."""
    v = imatrix.get(name + ".in")
    if v is None:
        return None
    v = np.maximum(v.astype(np.float64), 0)
    return np.maximum(v / max(v.mean(), 1e-30), floor).astype(np.float32)
