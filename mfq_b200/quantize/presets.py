"""Role-based mixed-width NINT presets ``S2-S .. S8``.

A preset names a base width; a handful of tensor roles get more bits because errors there cost more: the value
projection (few KV heads serve many query heads), the FFN down projection of the first layers, embeddings / output
head, shared experts and the small linear-attention control projections.  The schedule that picks "every third layer
plus both ends" is the one used by llama.cpp style K-quant mixes.  Behaviour parity:
``mfq/quantize/standard_presets.py:12-37`` (names and base widths) and ``:340-420`` (role rules) of the reference.
Roles are read off canonical tensor names (``model.block.N.attention.value.weight`` ...).
"""

from __future__ import annotations

import re
from dataclasses import dataclass

PRESETS = {"S2-S": 2, "S2-M": 2, "S3-S": 3, "S3-M": 3, "S3-L": 3, "S4-S": 4, "S4-M": 4, "S5-S": 5, "S5-M": 5, "S6": 6, "S8": 8}

_LAYER = re.compile(r"(?:^|\.)block\.(\d+)\.")
_NOT_QUANTIZED = ("norm.weight", ".router.weight", ".conv.weight", "shared_expert.router.weight", ".bias")
_CONTROL = {"alpha", "beta", "forget_a", "forget_b", "gate_a", "gate_b"}


def normalize_preset(name: str) -> str:
    p = name.strip().upper().replace("_", "-")
    if p not in PRESETS:
        raise ValueError(f"unsupported preset {name!r}; choose one of: {', '.join(PRESETS)}")
    return p


def tensor_role(name: str) -> str:
    """Coarse role of a canonical tensor name."""
    parts = name.split(".")
    if name in ("model.output.weight",):
        return "output"
    if name.endswith("token_embedding.weight"):
        return "embedding"
    if len(parts) >= 3 and parts[-3] == "linear_attention" and parts[-2] in _CONTROL:
        return "linear_control"
    if "shared_expert" in parts:
        return "shared_expert"
    if "experts" in parts:
        return "routed_expert"
    if name.endswith(("attention.value.weight", "attention.qkv.weight", "linear_attention.qkv.weight")):
        return "attention_v"
    if name.endswith("attention.key.weight"):
        return "attention_k"
    if name.endswith("attention.query.weight"):
        return "attention_q"
    if name.endswith(("attention.output.weight", "linear_attention.output.weight")):
        return "attention_output"
    if ".mlp.down" in name:
        return "ffn_down"
    if ".mlp.up" in name:
        return "ffn_up"
    if ".mlp.gate" in name:
        return "ffn_gate"
    return "other"


def quantizable(name: str, shape) -> bool:
    if not name.endswith(".weight") or len(shape) not in (2, 3):
        return False
    if len(shape) == 3 and "experts" not in name.split("."):
        return False
    return not any(marker in name for marker in _NOT_QUANTIZED)


def more_bits(index: int, count: int) -> bool:
    """First eighth, last eighth and every third layer in between."""
    if count <= 0:
        return False
    e = count // 8
    return index < e or index >= 7 * e or (index - e) % 3 == 2


@dataclass(frozen=True)
class Topology:
    layers: int
    heads: int
    kv_heads: int

    @property
    def gqa(self) -> int:
        return max(1, self.heads // max(1, self.kv_heads))


def select_bits(preset: str, name: str, topo: Topology, attention_index: int | None = None,
                attention_count: int | None = None) -> int:
    """NINT width of one tensor under ``preset``.  ``attention_index`` / ``attention_count`` number the layers that
    own a value projection (they differ from the layer index in hybrid models); they default to the layer index."""
    p = normalize_preset(preset)
    base = PRESETS[p]
    role = tensor_role(name)
    m = _LAYER.search(name)
    layer = int(m.group(1)) if m else 0
    n = max(1, topo.layers)
    ai = layer if attention_index is None else attention_index
    an = n if attention_count is None else attention_count
    if role == "linear_control" or role == "shared_expert":
        return 8
    if role in ("output", "embedding"):
        return 8 if p == "S8" else 6
    if role == "attention_v":
        table = {"S2-M": 4 if topo.gqa >= 4 else 3, "S2-S": 4 if topo.gqa >= 4 else base, "S3-M": 5 if ai < 2 else 4, "S3-L": 5,
                 "S4-M": 6 if more_bits(ai, an) else base, "S5-M": 6 if more_bits(ai, an) else base,
                 "S4-S": 5 if ai < 4 else base}
        return table.get(p, base)
    if role == "ffn_down":
        table = {"S2-M": 3, "S2-S": 4 if layer < n // 8 else base,
                 "S3-M": 5 if layer < n // 16 else (4 if more_bits(layer, n) else 3), "S3-L": 5,
                 "S4-M": 6 if more_bits(layer, n) else base, "S5-M": 6 if more_bits(layer, n) else base,
                 "S4-S": 5 if layer < n // 8 else base}
        return table.get(p, base)
    if role == "attention_output":
        return {"S2-M": 3, "S3-M": 4, "S3-L": 5}.get(p, base)
    return base


def plan(preset: str, tensors: dict[str, tuple], topo: Topology) -> dict[str, int | None]:
    """``{name: NINT width or None (kept as is)}`` for a whole checkpoint (``tensors`` maps name -> shape)."""
    owners = sorted({int(_LAYER.search(n).group(1)) for n in tensors if tensor_role(n) == "attention_v" and _LAYER.search(n)})
    rank = {layer: i for i, layer in enumerate(owners)}
    out: dict[str, int | None] = {}
    for name, shape in tensors.items():
        if not quantizable(name, shape):
            out[name] = None
            continue
        m = _LAYER.search(name)
        ai = rank.get(int(m.group(1))) if m else None
        out[name] = select_bits(preset, name, topo, ai, len(owners) or None)
    return out
