"""``model_graph.json``: the runtime-facing description of what a checkpoint contains.

The graph names the architecture and backbone, counts the layers of every component (text decoder, vision tower,
next-token predictor = MTP head), lists the optional components that are present and the capabilities they give, and
records the canonical tensor namespace.  A loader checks it before touching tensors, so a checkpoint with a component
the runtime cannot serve fails early with a clear message.  Same keys as the reference writes
(``mfq/architectures/tensor_schema.py:84-180``; parsed natively by ``cpp_runtime/core/mfq_model_graph.cpp``).
"""

from __future__ import annotations

import json
import re
from dataclasses import dataclass, field

SCHEMA_VERSION = 1
NAMESPACE = "mfq.tensor"
ASSET_NAME = "model_graph.json"
_ROOTS = ("model", "vision", "predictor", "audio", "tts", "runtime")
_CONTRACT = {
    "vision": {"kind": "vision", "implementation": "grid_vit", "policy": "optional", "capabilities": ("vision",)},
    "predictor": {"kind": "predictor", "implementation": "next_token_prediction", "policy": "optional",
                  "capabilities": ("speculative_prediction",)},
    "audio": {"kind": "audio_input", "implementation": "audio_encoder", "policy": "optional", "capabilities": ("audio_input",)},
    "tts": {"kind": "audio_output", "implementation": "tts_decoder", "policy": "optional", "capabilities": ("audio_output",)},
    "runtime": {"kind": "runtime", "implementation": "runtime", "policy": "optional", "capabilities": ()},
}
_OPTIONAL_KEY = {"vision": "vision", "predictor": "predictor", "audio": "audio_input", "tts": "audio_output", "runtime": "duplex"}
_LAYER = re.compile(r"^(model|vision|predictor)\.block\.(\d+)\.")


def backbone_of(config: dict) -> str:
    """Backbone family of a config: hybrid (linear + full attention), mixture of experts, or dense decoder."""
    if config.get("full_attention_interval") or config.get("linear_v_heads"):
        return "hybrid_gdn_moe"
    if config.get("kv_lora_rank"):
        return "mla_moe"
    if config.get("num_experts"):
        return "moe_decoder"
    return "dense_decoder"


def build_graph(config: dict, tensor_names, architecture: str = "mfq_b200_decoder") -> dict:
    names = list(tensor_names)
    roots = [r for r in _ROOTS if any(n.startswith(r + ".") for n in names)]
    if "model" not in roots:
        roots.insert(0, "model")
    layers = {"model": set(), "vision": set(), "predictor": set()}
    for n in names:
        m = _LAYER.match(n)
        if m:
            layers[m.group(1)].add(int(m.group(2)))
    backbone = backbone_of(config)
    components = [{"kind": "text", "tensor_root": "model", "implementation": backbone, "policy": "decoder"}]
    capabilities = ["text"]
    for r in roots:
        if r == "model":
            continue
        c = _CONTRACT[r]
        components.append({"kind": c["kind"], "tensor_root": r, "implementation": c["implementation"], "policy": c["policy"]})
        capabilities += list(c["capabilities"])
    return {
        "schema_version": SCHEMA_VERSION, "architecture": architecture, "graph": {"kind": "causal_lm", "backbone": backbone},
        "topology": {"text_layers": max(len(layers["model"]), int(config.get("num_layers", 0) or 0)),
                     "vision_layers": len(layers["vision"]), "predictor_layers": len(layers["predictor"])},
        "optional_components": {key: root in roots for root, key in _OPTIONAL_KEY.items()},
        "capabilities": capabilities, "components": components,
        "canonical_naming": {"namespace": NAMESPACE, "version": SCHEMA_VERSION, "component_roots": roots},
    }


def to_bytes(graph: dict) -> bytes:
    return json.dumps(graph, ensure_ascii=False, separators=(",", ":"), sort_keys=True).encode("utf-8")


@dataclass
class ModelGraph:
    architecture: str
    backbone: str
    text_layers: int
    vision_layers: int = 0
    predictor_layers: int = 0
    capabilities: tuple[str, ...] = ("text",)
    component_roots: tuple[str, ...] = ("model",)
    raw: dict = field(default_factory=dict)

    def has(self, capability: str) -> bool:
        return capability in self.capabilities

    def unsupported(self, served=("text", "speculative_prediction")) -> list[str]:
        """Capabilities of the checkpoint that a runtime serving only ``served`` would have to ignore."""
        return [c for c in self.capabilities if c not in served]


def parse_graph(data: bytes | str | dict) -> ModelGraph:
    g = data if isinstance(data, dict) else json.loads(data)
    if int(g.get("schema_version", 0)) != SCHEMA_VERSION:
        raise ValueError(f"model graph schema {g.get('schema_version')!r} is not supported (expected {SCHEMA_VERSION})")
    kind = (g.get("graph") or {}).get("kind")
    if kind != "causal_lm":
        raise ValueError(f"model graph kind {kind!r} is not a causal language model")
    naming = g.get("canonical_naming") or {}
    if naming.get("namespace", NAMESPACE) != NAMESPACE:
        raise ValueError(f"tensor namespace {naming.get('namespace')!r} is not {NAMESPACE!r}")
    topo = g.get("topology") or {}
    roots = tuple(naming.get("component_roots") or [c.get("tensor_root") for c in g.get("components", [])] or ["model"])
    if "model" not in roots:
        raise ValueError("a model graph needs a text component")
    return ModelGraph(str(g.get("architecture", "")), str(g["graph"].get("backbone", "")), int(topo.get("text_layers", 0)),
                      int(topo.get("vision_layers", 0)), int(topo.get("predictor_layers", 0)),
                      tuple(g.get("capabilities") or ("text",)), roots, g)
