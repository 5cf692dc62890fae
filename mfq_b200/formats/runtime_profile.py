"""Embedded sampling defaults: the ``runtime.sampling.v1`` header entry of a checkpoint.

A checkpoint may carry the sampling defaults its family was validated with (temperature, top-p, draft depth ...);
the server merges them under the request's own parameters.  Resolution order, most specific first: the profile
embedded in the file, the generation config shipped as a Hugging Face asset, the architecture registry, built-in
defaults.  Reference: ``mfq/formats/runtime_profile.py:53-395`` and ``docs/runtime/sampling-profiles.md``.
"""

from __future__ import annotations

import json
from typing import Any, Mapping

SCHEMA = "mfq.runtime.sampling"
VERSION = 1
HEADER_KEY = "runtime.sampling.v1"

_CHAT_KEYS = {"temperature", "top_k", "top_p", "presence_penalty", "frequency_penalty", "repetition_penalty", "max_tokens",
              "enable_thinking", "enable_mtp", "mtp_max_draft_tokens", "seed"}
BUILTIN = {"temperature": 0.0, "top_k": 0, "top_p": 1.0, "presence_penalty": 0.0, "frequency_penalty": 0.0,
           "repetition_penalty": 1.0, "max_tokens": 256, "enable_mtp": False, "mtp_max_draft_tokens": 3}
_REGISTRY: dict[str, dict[str, Any]] = {
    "llama": {"temperature": 0.6, "top_p": 0.9},
    "qwen3_next": {"temperature": 0.7, "top_k": 20, "top_p": 0.8, "enable_mtp": True, "mtp_max_draft_tokens": 3},
    "deepseek_v3": {"temperature": 0.6, "top_p": 0.95, "enable_mtp": True, "mtp_max_draft_tokens": 1},
}


def make_profile(chat: Mapping[str, Any], source: str) -> dict[str, Any]:
    unknown = set(chat) - _CHAT_KEYS
    if unknown:
        raise ValueError(f"unknown sampling keys: {sorted(unknown)}")
    return {"schema": SCHEMA, "version": VERSION, "chat": dict(chat), "provenance": {"source": source}}


def validate(profile: Mapping[str, Any]) -> dict[str, Any]:
    if profile.get("schema") != SCHEMA or int(profile.get("version", 0)) != VERSION:
        raise ValueError("not a runtime.sampling.v1 profile")
    chat = dict(profile.get("chat", {}))
    if set(chat) - _CHAT_KEYS:
        raise ValueError(f"unknown sampling keys: {sorted(set(chat) - _CHAT_KEYS)}")
    if not 0.0 <= float(chat.get("top_p", 1.0)) <= 1.0 or float(chat.get("temperature", 0.0)) < 0.0:
        raise ValueError("sampling profile out of range")
    return {"schema": SCHEMA, "version": VERSION, "chat": chat, "provenance": dict(profile.get("provenance", {}))}


def from_generation_config(text: str | bytes) -> dict[str, Any] | None:
    """Profile from a Hugging Face ``generation_config.json`` (only the keys it actually sets)."""
    cfg = json.loads(text)
    if cfg.get("do_sample") is False:
        return make_profile({"temperature": 0.0}, "hf-generation-config")
    chat = {k: cfg[k] for k in ("temperature", "top_k", "top_p", "repetition_penalty") if cfg.get(k) is not None}
    return make_profile(chat, "hf-generation-config") if chat else None


def resolve(header_extra: Mapping[str, Any] | None = None, assets: Mapping[str, bytes] | None = None,
            architecture: str | None = None) -> dict[str, Any]:
    """Effective chat defaults + where they came from."""
    out, source = dict(BUILTIN), "builtin"
    if architecture and architecture in _REGISTRY:
        out.update(_REGISTRY[architecture])
        source = f"architecture-registry:{architecture}"
    gen = (assets or {}).get("hf/generation_config.json")
    if gen:
        prof = from_generation_config(gen)
        if prof:
            out.update(prof["chat"])
            source = "hf-generation-config"
    embedded = (header_extra or {}).get(HEADER_KEY)
    if embedded:
        out.update(validate(embedded)["chat"])
        source = "embedded"
    return {"chat": out, "source": source}


def merge_request(defaults: Mapping[str, Any], request: Mapping[str, Any]) -> dict[str, Any]:
    """Request values win; ``None`` means "not given"."""
    out = dict(defaults)
    out.update({k: v for k, v in request.items() if v is not None and k in _CHAT_KEYS})
    return out
