"""Per-expert-projection precision: seeded balanced allocation and MFE assembly.

``balanced_expert_mix`` reproduces the reference's deterministic fixture rule
(``mfq/tools/quantize_hf_to_mfq.py:2598-2619``): every routed projection tensor gets
its own shuffle of ``arange(n_experts) % n_profiles`` drawn from
``SeedSequence((seed, n_experts, *utf8(name)))``, so each family serves the same
number of experts and the placement is a pure function of (seed, tensor name).
``quantize_expertwise`` then groups experts by profile into MFE pools.
"""

from __future__ import annotations

from dataclasses import dataclass

import numpy as np

from ..formats.mfe import MfePool, MfeTensor
from ..formats.nint import NintSpec
from ..formats.nvq import NvqSpec
from .fp8_block import quantize_fp8_block
from .mxfp4 import quantize_mxfp4
from .nint import quantize_nint
from .nvq import quantize_nvq

DEFAULT_MIX_SEED = 20260908

# nominal NINT presets by width: (groupsize, sub_bits), mirroring the k-quant-style defaults
_NINT_PRESETS = {2: (16, 4), 3: (16, 6), 4: (24, 6), 5: (28, 7), 6: (16, 8), 8: (32, 8), 1: (16, 4), 7: (32, 8)}
_NVQ_FAMILIES = {"NVQ2": "e8_256", "NVQ3": "d4_256", "NVQ3-512": "d4_512", "NVQ3-L": "d4_1024",
                 "NVQ2-1024": "e8_1024", "NVQ2-4096": "e8_4096"}

# joint scale/codebook-state lattice families: base grid, banks, learned scale table, storage layout
_NVQ_JSC_FAMILIES = {"NVQ2J": ("e8_256", 2, True, "streams"), "NVQ2J-L": ("e8_1024", 2, True, "streams"),
                     "NVQ2J-XL": ("e8_4096", 4, True, "group64"), "NVQ3J": ("d4_256", 2, False, "streams"),
                     "NVQ3J-512": ("d4_512", 2, False, "streams"), "NVQ3J-L": ("d4_1024", 2, False, "streams")}

__all__ = ["ExpertProfile", "parse_profiles", "balanced_expert_mix", "quantize_expertwise", "quantize_matrix",
           "DEFAULT_MIX_SEED"]


@dataclass(frozen=True)
class ExpertProfile:
    family: str  # "NINT4", "NVQ3", "MXFP4", "FP8", "BF16"
    nint: NintSpec | None = None
    nvq: NvqSpec | None = None

    @property
    def nominal_bpw(self) -> float:
        if self.nint is not None:
            return self.nint.bpw(4096)
        if self.nvq is not None:
            return self.nvq.bpw(4096, out=4096)
        if self.family in _NVQ_JSC_FAMILIES:
            return NvqSpec(_NVQ_JSC_FAMILIES[self.family][0]).bpw(4096, out=4096)
        return {"MXFP4": 4.25, "FP8": 8.0, "BF16": 16.0, "NPQ0-S": 0.84, "NPQ0-L": 1.0, "NVQ1-L": 1.55, "NVQ1-L-S4": 1.59,
                "NVQ1-S": 1.34, "NEPQ0-S": 0.88, "NEPQ0-L": 1.04, "NEPQ1-S": 1.42, "NEPQ1-L": 1.63, "NEPQ0-A": 0.96,
                "NEPQ1-A": 1.61}[self.family]


def parse_profiles(text: str) -> tuple[ExpertProfile, ...]:
    names = [p.strip().upper() for p in text.split(",") if p.strip()]
    if len(set(names)) != len(names):
        raise ValueError("duplicate precision families in the expert mix")
    out = []
    for name in names:
        if name.startswith("NINT") and name[4:].isdigit():
            bits = int(name[4:])
            gs, k = _NINT_PRESETS[bits]
            out.append(ExpertProfile(name, nint=NintSpec(bits, gs, k)))
        elif name in _NVQ_FAMILIES:
            out.append(ExpertProfile(name, nvq=NvqSpec(_NVQ_FAMILIES[name])))
        elif name in _NVQ_JSC_FAMILIES:
            out.append(ExpertProfile(name))
        elif name in ("MXFP4", "FP8", "BF16", "NPQ0-S", "NPQ0-L", "NVQ1-L", "NVQ1-L-S4", "NVQ1-S", "NEPQ0-S", "NEPQ0-L", "NEPQ1-S",
                      "NEPQ1-L", "NEPQ0-A", "NEPQ1-A"):
            out.append(ExpertProfile(name))
        else:
            raise ValueError(f"unsupported expert precision {name!r}")
    return tuple(out)


def balanced_expert_mix(tensor_name: str, n_experts: int, n_profiles: int, seed: int = DEFAULT_MIX_SEED) -> np.ndarray:
    """Profile index per expert for one projection tensor (balanced, reproducible)."""
    idx = np.arange(n_experts, dtype=np.int64) % n_profiles
    rng = np.random.default_rng(np.random.SeedSequence((int(seed), int(n_experts), *tensor_name.encode("utf-8"))))
    rng.shuffle(idx)
    return idx


def quantize_matrix(w, profile: ExpertProfile, device="cpu", importance=None):
    """One ``[out, in]`` (or stacked) matrix -> family tensor object (``importance``: per-input weights, NINT only)."""
    if profile.nint is not None:
        return quantize_nint(w, profile.nint, device=device, importance=importance)
    if profile.nvq is not None:
        return quantize_nvq(w, profile.nvq, device=device)
    if profile.family == "MXFP4":
        return quantize_mxfp4(w, device=device)
    if profile.family == "FP8":
        return quantize_fp8_block(w, device=device)
    if profile.family in ("NPQ0-S", "NPQ0-L"):
        from ..formats.npq0 import quantize_npq0
        return quantize_npq0(np.asarray(w, dtype=np.float32), profile.family)
    if profile.family.startswith("NVQ1-"):
        from ..formats.nvq1 import quantize_nvq1
        w = np.asarray(w, dtype=np.float32)
        return quantize_nvq1(w, profile.family, axis=w.ndim - 2, importance=importance, device=str(device))
    if profile.family in _NVQ_JSC_FAMILIES:
        from .nvq_jsc import quantize_nvq_jsc
        grid, banks, learned, layout = _NVQ_JSC_FAMILIES[profile.family]
        w = np.asarray(w, dtype=np.float32)
        return quantize_nvq_jsc(w, grid, banks=banks, axis=w.ndim - 2, importance=importance, learn_scales=learned,
                                storage_layout=layout, device=device)
    if profile.family.startswith("NEPQ"):
        from ..formats.nepq import quantize_nepq
        w = np.asarray(w, dtype=np.float32)
        return quantize_nepq(w if w.ndim == 3 else w[None], profile.family, device=str(device))  # the experts share one table pool
    if profile.family == "BF16":
        from ..formats.dense import to_bf16
        return to_bf16(np.asarray(w, dtype=np.float32))
    raise ValueError(profile.family)


def quantize_expertwise(weights, assignment: np.ndarray, profiles: tuple[ExpertProfile, ...], device="cpu") -> MfeTensor:
    """``weights [experts, out, in]`` + profile index per expert -> MFE tensor (one pool per profile used)."""
    w = np.asarray(weights, dtype=np.float32)
    n, out, k = w.shape
    pools = []
    for pi, profile in enumerate(profiles):
        ids = np.flatnonzero(assignment == pi).astype(np.int32)
        if ids.size:
            stacked = profile.family.startswith("NEPQ")  # coded as [experts, out, K]: bank ids and anchors are per expert row
            pools.append(MfePool(ids, quantize_matrix(w[ids] if stacked else w[ids].reshape(ids.size * out, k), profile, device)))
    return MfeTensor((n, out, k), tuple(pools))
