"""MoE cache profile: which experts were hot, saved at shutdown and used to warm the HBM arena at the next start.

With routed experts behind an HBM arena (``--moe-gpu-cache-gb`` / ``--moe-gpu-cache-slots``) the first requests after a
start pay an upload for every expert they touch.  Expert popularity is stable for a given deployment, so the decayed
per-expert heat that each layer's :class:`~mfq_b200.engine.expert_residency.ExpertResidency` gathers is written to a
small JSON file (``--moe-cache-profile PATH``) and, at the next start, the hottest experts of every layer are uploaded
before the server accepts traffic.  A profile from another model (layer count or expert count differs) is ignored.

Reference: ``cpp_runtime/core/include/mfq/moe_cache_profile.h`` and the runtime flag ``--moe-cache-profile``.
"""

from __future__ import annotations

import json
import os
from pathlib import Path

FORMAT = "mfq.moe-cache-profile.v1"


def _residencies(model) -> dict[int, object]:
    out = {}
    for i, layer in enumerate(model.w.layers):
        ffn = getattr(layer, "moe", None)
        if ffn is not None and getattr(ffn, "residency", None) is not None:
            out[i] = ffn.residency
    return out


def collect(model, name: str = "") -> dict:
    for r in _residencies(model).values():
        r.absorb_heat()  # usage counted on the device by graph-captured steps
    layers = {str(i): {"heat": [round(float(h), 4) for h in r.heat], "slots": r.slots, "stats": dict(r.stats)}
              for i, r in _residencies(model).items()}
    return {"format": FORMAT, "model": name, "rank": getattr(model.w, "tp_rank", 0), "layers": layers}


def save(path, profile: dict) -> None:
    p = Path(path)
    p.parent.mkdir(parents=True, exist_ok=True)
    tmp = p.with_name(p.name + f".tmp-{os.getpid()}")
    tmp.write_text(json.dumps(profile))
    os.replace(tmp, p)


def load(path) -> dict | None:
    try:
        doc = json.loads(Path(path).read_text())
    except (OSError, ValueError):
        return None
    return doc if doc.get("format") == FORMAT else None


def apply(model, profile: dict | None) -> int:
    """Warm every layer's arena from ``profile``; returns the number of experts uploaded (0 if it does not fit)."""
    res = _residencies(model)
    if not profile or not res or set(profile.get("layers", {})) != {str(i) for i in res}:
        return 0
    if any(len(profile["layers"][str(i)]["heat"]) != r.n for i, r in res.items()):
        return 0
    return sum(len(r.warm(profile["layers"][str(i)]["heat"])) for i, r in res.items())
