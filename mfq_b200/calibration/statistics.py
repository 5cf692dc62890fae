"""Activation and Fisher statistics of every linear layer over a calibration corpus.

For a projection ``y = W x`` and a next-token loss ``L`` the squared gradient of row ``r`` of ``W`` summed over its columns
is ``(dL/dy_r)^2 * |x|^2``.  Two vectors per projection and split are collected:

* ``input second moment [columns]`` -- mean of ``x_c^2`` over the tokens the layer saw (what importance-weighted weight
  quantizers use as column weights), and
* ``row Fisher [rows]`` -- mean over scored positions of ``(dL/dy_r)^2 * |x|^2``, the diagonal Fisher information of the
  layer summed along each output row (what precision allocation uses to compare layers and rows).

The model is the fp32 restatement (:class:`mfq_b200.models.moe_lm.MoeLM`, pure torch, so autograd gives the output
gradients).  Routed experts are recorded per expert as ``<tensor>#<e>`` with their input statistics and exposure
counts only; their Fisher vectors are left at the floor.

File: one ``.npz`` -- arrays ``entry_NNNN_{train,validation}_{input,fisher}`` plus ``__metadata_json__`` (UTF-8 JSON:
``format`` ``mfq.calibration-statistics.v1``, run metadata, and per entry its array prefix, target description and the
four counts).  Zeros are floored at 1e-12 of the array's positive mean on save, as consumers divide by these values.

Reference: ``mfq/calibration/statistics.py`` (``TensorStatistics`` :40, ``save_statistics`` :76, ``load_statistics`` :124,
``Qwen35StatisticsCollector`` :177, ``_collect_fisher_statistics`` :585) -- same file layout and quantities; the reference
streams one bf16 layer of a Hugging Face model at a time through forward/backward hooks.
"""

from __future__ import annotations

import json
import os
from dataclasses import asdict, dataclass, field
from pathlib import Path
from typing import Any, Mapping

import numpy as np
import torch

FORMAT = "mfq.calibration-statistics.v1"
_META = "__metadata_json__"


@dataclass(frozen=True)
class LinearTarget:
    name: str
    rows: int
    columns: int
    group: str = ""   # "attention" / "mlp" / "expert" / "head"
    role: str = ""    # query / key / value / output / gate / up / down / ...


@dataclass
class TensorStatistics:
    target: LinearTarget
    train_input_second_moment: np.ndarray
    validation_input_second_moment: np.ndarray
    train_row_fisher: np.ndarray
    validation_row_fisher: np.ndarray
    train_input_count: int = 0
    validation_input_count: int = 0
    train_fisher_probes: int = 0
    validation_fisher_probes: int = 0


@dataclass
class CalibrationStatistics:
    path: Path
    entries: dict[str, TensorStatistics]
    metadata: dict[str, Any] = field(default_factory=dict)

    def require(self, name: str) -> TensorStatistics:
        if name not in self.entries:
            raise KeyError(f"calibration statistics have no tensor {name!r}")
        return self.entries[name]

    def as_imatrix(self, split: str = "train") -> dict[str, np.ndarray]:
        """The input statistics in the ``<name>.in`` / ``<name>.count`` form the quantizers read."""
        out = {}
        for name, e in self.entries.items():
            out[name + ".in"] = getattr(e, f"{split}_input_second_moment")
            out[name + ".count"] = np.array(getattr(e, f"{split}_input_count"), dtype=np.int64)
        return out


def _floored(v, label: str) -> np.ndarray:
    a = np.asarray(v, dtype=np.float64).reshape(-1)
    if not a.size or not np.isfinite(a).all() or (a < 0).any():
        raise ValueError(f"invalid non-negative statistic for {label}")
    pos = a[a > 0]
    floor = max(float(pos.mean()) * 1e-12, float(np.finfo(np.float32).tiny)) if pos.size else float(np.finfo(np.float32).tiny)
    return np.ascontiguousarray(np.maximum(a, floor), dtype=np.float32)


def save_statistics(path, entries: Mapping[str, TensorStatistics], metadata: Mapping[str, Any]) -> None:
    out = Path(path)
    if out.exists():
        raise FileExistsError(f"calibration statistics already exist: {out}")
    if not entries:
        raise ValueError("cannot save empty calibration statistics")
    arrays: dict[str, np.ndarray] = {}
    doc_entries: dict[str, Any] = {}
    for i, (name, e) in enumerate(sorted(entries.items())):
        prefix = f"entry_{i:04d}"
        for suffix, raw in (("train_input", e.train_input_second_moment), ("validation_input", e.validation_input_second_moment),
                            ("train_fisher", e.train_row_fisher), ("validation_fisher", e.validation_row_fisher)):
            arrays[f"{prefix}_{suffix}"] = _floored(raw, f"{name}/{suffix}")
        doc_entries[name] = {"prefix": prefix, "target": asdict(e.target),
                             "counts": {"train_input": int(e.train_input_count), "validation_input": int(e.validation_input_count),
                                        "train_fisher_probes": int(e.train_fisher_probes),
                                        "validation_fisher_probes": int(e.validation_fisher_probes)}}
    doc = {"format": FORMAT, "metadata": dict(metadata), "entries": doc_entries}
    arrays[_META] = np.frombuffer(json.dumps(doc, ensure_ascii=False, separators=(",", ":")).encode("utf-8"), dtype=np.uint8).copy()
    out.parent.mkdir(parents=True, exist_ok=True)
    tmp = out.with_suffix(out.suffix + ".tmp")
    with tmp.open("wb") as f:
        np.savez_compressed(f, **arrays)
    os.replace(tmp, out)


def load_statistics(path) -> CalibrationStatistics:
    p = Path(path)
    with np.load(p, allow_pickle=False) as z:
        if _META not in z.files:
            raise ValueError(f"calibration statistics have no metadata: {p}")
        doc = json.loads(z[_META].tobytes().decode("utf-8"))
        if doc.get("format") != FORMAT:
            raise ValueError(f"unsupported calibration statistics format: {doc.get('format')!r}")
        entries = {}
        for name, item in doc["entries"].items():
            known = {k: v for k, v in item["target"].items() if k in LinearTarget.__dataclass_fields__}
            target = LinearTarget(**known)
            arr = {s: np.asarray(z[f"{item['prefix']}_{s}"], dtype=np.float32)
                   for s in ("train_input", "validation_input", "train_fisher", "validation_fisher")}
            if arr["train_input"].shape != (target.columns,) or arr["train_fisher"].shape != (target.rows,):
                raise ValueError(f"statistic width mismatch for {name}")
            c = item["counts"]
            entries[name] = TensorStatistics(target, arr["train_input"], arr["validation_input"], arr["train_fisher"],
                                             arr["validation_fisher"], int(c["train_input"]), int(c["validation_input"]),
                                             int(c["train_fisher_probes"]), int(c["validation_fisher_probes"]))
    return CalibrationStatistics(p, entries, dict(doc.get("metadata", {})))


class _Accumulator:
    """Sums for one split: the ``observer`` hook of the fp32 model.  With ``fisher`` on, every observed output gets a
    gradient hook; the model must then run with gradients enabled and a loss must be back-propagated per window."""

    def __init__(self, fisher: bool) -> None:
        self.fisher = fisher
        self.sum_in: dict[str, torch.Tensor] = {}
        self.n_in: dict[str, int] = {}
        self.sum_fisher: dict[str, torch.Tensor] = {}
        self.n_fisher: dict[str, int] = {}
        self.shape: dict[str, tuple[int, int]] = {}

    def observe(self, name: str, x: torch.Tensor, y: torch.Tensor | None = None) -> None:
        x2 = x.detach().reshape(-1, x.shape[-1]).double()
        self.sum_in[name] = self.sum_in.get(name, 0) + (x2 * x2).sum(0)
        self.n_in[name] = self.n_in.get(name, 0) + x2.shape[0]
        if y is None:
            return
        self.shape[name] = (int(y.shape[-1]), int(x.shape[-1]))
        if self.fisher and y.requires_grad:
            energy = (x2 * x2).sum(-1, keepdim=True)  # |x|^2 per token

            def hook(g, name=name, energy=energy):
                g2 = g.detach().reshape(-1, g.shape[-1]).double()
                self.sum_fisher[name] = self.sum_fisher.get(name, 0) + (g2 * g2 * energy).sum(0)
                self.n_fisher[name] = self.n_fisher.get(name, 0) + int((g2.abs().sum(-1) > 0).sum())

            y.register_hook(hook)


def _group_role(name: str) -> tuple[str, str]:
    role = name.rsplit(".", 2)[-2] if name.endswith(".weight") else name.rsplit(".", 1)[-1]
    if "#" in name:
        return "expert", name.split("#")[0].rsplit(".", 2)[-2]
    if ".attention." in name:
        return "attention", role
    if ".mlp." in name:
        return "mlp", role
    return "head", role


def collect_statistics(cfg, tensors: Mapping[str, Any], corpus, output, *, device: str = "cpu",
                       train_input_tokens: int = 1 << 16, validation_input_tokens: int = 1 << 14,
                       train_fisher_tokens: int = 1 << 14, validation_fisher_tokens: int = 1 << 12,
                       window: int | None = None, seed: int = 0, progress=None) -> CalibrationStatistics:
    """Run the corpus' windows through the fp32 model (``cfg`` a :class:`MoeConfig`, ``tensors`` its dequantized
    weights): the first ``*_fisher_tokens`` of every split with a backward pass (their inputs count towards the input
    statistics as well), the rest up to ``*_input_tokens`` forward only.  Writes ``output`` and returns what it wrote."""
    from ..models.moe_lm import MoeLM
    dev = torch.device(device)
    w = {k: torch.as_tensor(np.asarray(v, dtype=np.float32)).to(dev) for k, v in tensors.items()}
    acc = {s: _Accumulator(fisher=True) for s in ("train", "validation")}
    budgets = {"train": (train_input_tokens, train_fisher_tokens), "validation": (validation_input_tokens, validation_fisher_tokens)}
    losses = {}
    for split in ("train", "validation"):
        a = acc[split]
        model = MoeLM(cfg, w, observer=a.observe)
        # the embedding output must carry a gradient so that every later activation does
        embed = w["model.token_embedding.weight"]
        in_budget, fisher_budget = budgets[split]
        seen = scored = 0
        total_loss = 0.0
        for toks, mask in corpus.iter_chunks(split, max_tokens=in_budget):
            if window:
                toks, mask = toks[:window], mask[:window]
            ids = torch.from_numpy(np.ascontiguousarray(toks)).to(dev)
            want_fisher = seen < fisher_budget
            a.fisher = want_fisher
            model.reset()
            if want_fisher:
                leaf = embed.detach().clone().requires_grad_(True)
                model.w = {**w, "model.token_embedding.weight": leaf}
                with torch.enable_grad():
                    logits = model.forward(ids)
                    m = torch.from_numpy(np.ascontiguousarray(mask[1:]).astype(np.bool_)).to(dev)
                    if int(m.sum()) > 0:
                        lp = torch.log_softmax(logits[:-1].float(), -1).gather(1, ids[1:, None].long())[:, 0]
                        # per-position gradients are summed, not averaged: each scored position is one Fisher probe
                        loss = -(lp * m).sum()
                        loss.backward()
                        total_loss += float(loss.detach())
                        scored += int(m.sum())
                model.w = w
            else:
                with torch.no_grad():
                    model.forward(ids)
            seen += int(toks.size)
            if progress:
                progress(split, seen, in_budget)
        losses[split] = total_loss / max(1, scored)
    names = sorted(set(acc["train"].sum_in) | set(acc["validation"].sum_in))
    entries = {}
    for name in names:
        tr, va = acc["train"], acc["validation"]
        cols = int((tr.sum_in.get(name) if name in tr.sum_in else va.sum_in[name]).numel())
        rows = (tr.shape.get(name) or va.shape.get(name) or (0, cols))[0]
        if rows == 0:  # routed experts observe inputs only: rows from the stacked weight
            base, _, e = name.partition("#")
            rows = int(np.asarray(tensors[base]).shape[1]) if base in tensors else 1

        def mean(sums, counts, size):
            if name not in sums:
                return np.zeros(size)
            return (sums[name] / max(1, counts.get(name, 1))).cpu().numpy()

        group, role = _group_role(name)
        entries[name] = TensorStatistics(
            LinearTarget(name, rows, cols, group, role),
            mean(tr.sum_in, tr.n_in, cols), mean(va.sum_in, va.n_in, cols),
            mean(tr.sum_fisher, tr.n_fisher, rows), mean(va.sum_fisher, va.n_fisher, rows),
            tr.n_in.get(name, 0), va.n_in.get(name, 0), tr.n_fisher.get(name, 0), va.n_fisher.get(name, 0))
    meta = {"seed": int(seed), "device": str(dev), "corpus": {"path": str(corpus.root), "token_sha256": corpus.manifest.get("token_sha256")},
            "budgets": {s: {"input_tokens": b[0], "fisher_tokens": b[1]} for s, b in budgets.items()},
            "mean_scored_loss": losses, "model": {"layers": cfg.num_layers, "hidden_size": cfg.hidden_size, "vocab_size": cfg.vocab_size}}
    save_statistics(output, entries, meta)
    return load_statistics(output)
