"""Quantization recipes: per-tensor precisions taken from a GGUF file's tensor table, or from a JSON rule list.

A *recipe GGUF* is any GGUF of the same architecture that somebody already quantized to taste (the usual mixed K-quant
files): only its tensor TABLE is read -- names and ggml types, no payload -- and each tensor's type becomes the NINT
width of the same tensor here (``Q4_K`` -> NINT4, ``Q6_K`` -> NINT6, ``Q8_0`` -> NINT8, ``F16 / BF16 / F32`` -> keep
in bf16 ...).  A JSON recipe is a list of ``{"match": <regex on the canonical name>, "bits": 2..8 | null}`` rules, first
match wins, plus a ``"default"``.  Both give the ``widths`` plan that ``quantize_tensors`` takes.

Reference: ``mfq quantize --recipe RECIPE.gguf`` (``docs/cli/quantize.md``: "Mixed GGUF recipe").
"""

from __future__ import annotations

import json
import re
from pathlib import Path

# ggml type id -> NINT width (None: leave in bf16).  K-quants and I-quants map to the NINT width of the same nominal bits.
GGML_WIDTH = {
    0: None, 1: None, 30: None,             # F32, F16, BF16
    2: 4, 3: 4, 6: 5, 7: 5, 8: 8, 9: 8,     # Q4_0 Q4_1 Q5_0 Q5_1 Q8_0 Q8_1
    10: 2, 11: 3, 12: 4, 13: 5, 14: 6, 15: 8,  # Q2_K Q3_K Q4_K Q5_K Q6_K Q8_K
    16: 2, 17: 2, 18: 3, 19: 2, 20: 4, 21: 3, 22: 2, 23: 4, 29: 2,  # IQ2_XXS IQ2_XS IQ3_XXS IQ1_S IQ4_NL IQ3_S IQ2_S IQ4_XS IQ1_M
}


def widths_from_gguf(path, tensor_names) -> dict[str, int | None]:
    """``tensor_names``: canonical names of the model being quantized.  Stacked expert tensors take the width of the
    recipe's stacked (``ffn_*_exps``) tensor."""
    from ..formats.gguf import GgufFile, canonical_name
    table = GgufFile(path).tensors
    plan: dict[str, int | None] = {}
    unknown = set()
    for name, info in table.items():
        cname = canonical_name(name)
        if cname is None:
            continue
        if info.ggml_type not in GGML_WIDTH:
            unknown.add(info.ggml_type)
            continue
        plan[cname] = GGML_WIDTH[info.ggml_type]
    if unknown:
        raise ValueError(f"{path}: ggml tensor types {sorted(unknown)} have no NINT counterpart")
    wanted = set(tensor_names)
    return {k: v for k, v in plan.items() if k in wanted}


def widths_from_rules(doc: dict, tensor_names) -> dict[str, int | None]:
    rules = [(re.compile(r["match"]), r.get("bits")) for r in doc.get("rules", [])]
    for _rx, bits in rules:
        if bits is not None and not 2 <= int(bits) <= 8:
            raise ValueError(f"recipe: bits must be 2..8 or null, not {bits!r}")
    plan = {}
    for name in tensor_names:
        for rx, bits in rules:
            if rx.search(name):
                plan[name] = None if bits is None else int(bits)
                break
        else:
            if "default" in doc:
                plan[name] = None if doc["default"] is None else int(doc["default"])
    return plan


def load_recipe(path, tensor_names) -> dict[str, int | None]:
    p = Path(path)
    if p.suffix == ".gguf":
        return widths_from_gguf(p, tensor_names)
    return widths_from_rules(json.loads(p.read_text()), tensor_names)


def parse_size(text: str) -> int:
    """``"500M"`` / ``"4G"`` / ``"1048576"`` -> bytes."""
    m = re.fullmatch(r"\s*(\d+(?:\.\d+)?)\s*([kKmMgGtT]?)[iI]?[bB]?\s*", text)
    if not m:
        raise ValueError(f"cannot read a size from {text!r} (use e.g. 500M or 4G)")
    return int(float(m[1]) * 1024 ** " kmgt".index(m[2].lower() or " "))
