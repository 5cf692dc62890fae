"""Embedded sampling defaults: the ``runtime.sampling.v1`` header entry of a checkpoint.

A checkpoint may carry the sampling defaults its family was validated with (temperature, top-p, draft depth ...);
the server merges them under the request's own parameters.  Resolution order, most specific first: a sidecar file
beside the checkpoint (``<file>.runtime.json``; for shards also ``<family>.runtime.json``, which the exact file's
sidecar overrides), the profile embedded in the file, the generation config shipped as a Hugging Face asset, the
architecture registry, built-in defaults.  A profile has up to three sections -- ``chat`` (what this server samples
with), ``duplex`` and ``tts`` (carried and type-checked for the speech models of the reference, not interpreted
here) -- and a ``provenance``.  ``mfq quantize`` writes the profile of a new checkpoint with
:func:`profile_for_new_checkpoint`: registry entry of the source's architecture, then its ``generation_config.json``,
then an ``mfq-runtime.json`` found in the source directory, then ``--runtime-profile``; nothing is invented when none
of them says anything.  Reference: ``mfq/formats/runtime_profile.py:17-395`` and ``docs/runtime/sampling-profiles.md``.
"""

from __future__ import annotations

import json
import re
from pathlib import Path
from typing import Any, Mapping

SCHEMA = "mfq.runtime.sampling"
VERSION = 1
HEADER_KEY = "runtime.sampling.v1"

BUILTIN = {"temperature": 0.0, "top_k": 0, "top_p": 1.0, "presence_penalty": 0.0, "frequency_penalty": 0.0,
           "repetition_penalty": 1.0, "max_tokens": 256, "enable_mtp": False, "mtp_max_draft_tokens": 3}
_REGISTRY: dict[str, dict[str, Any]] = {
    "llama": {"temperature": 0.6, "top_p": 0.9},
    "qwen3_next": {"temperature": 0.7, "top_k": 20, "top_p": 0.8, "enable_mtp": True, "mtp_max_draft_tokens": 3},
    "deepseek_v3": {"temperature": 0.6, "top_p": 0.95, "enable_mtp": True, "mtp_max_draft_tokens": 1},
}


_FIELDS: dict[str, dict[str, type]] = {
    "chat": {"max_tokens": int, "temperature": float, "top_k": int, "top_p": float, "presence_penalty": float,
             "frequency_penalty": float, "repetition_penalty": float, "enable_thinking": bool, "enable_mtp": bool,
             "mtp_max_draft_tokens": int, "seed": int},
    "duplex": {"system_prompt": str, "decode_mode": str, "temperature": float, "top_k": int, "top_p": float,
               "text_repetition_penalty": float, "text_repetition_window_size": int, "length_penalty": float,
               "listen_prob_scale": float, "force_listen_count": int, "max_new_speak_tokens_per_chunk": int},
    "tts": {"temperature": float, "repetition_penalty": float, "token2wav_steps": int},
}
_RANGES = {"temperature": (0.0, None), "top_p": (0.0, 1.0), "top_k": (0, None), "max_tokens": (1, None),
           "repetition_penalty": (0.0, None), "text_repetition_penalty": (0.0, None), "mtp_max_draft_tokens": (0, 16),
           "token2wav_steps": (1, None), "text_repetition_window_size": (0, None), "force_listen_count": (0, None),
           "max_new_speak_tokens_per_chunk": (1, None), "listen_prob_scale": (0.0, None)}


def _typed(section: str, key: str, value: Any) -> Any:
    kind = _FIELDS[section][key]
    if kind is bool:
        if not isinstance(value, bool):
            raise ValueError(f"{section}.{key} must be true or false")
        return value
    if kind is str:
        if not isinstance(value, str):
            raise ValueError(f"{section}.{key} must be a string")
        return value
    if isinstance(value, bool) or not isinstance(value, (int, float)):
        raise ValueError(f"{section}.{key} must be a number")
    if kind is int:
        if float(value) != int(value):
            raise ValueError(f"{section}.{key} must be an integer")
        value = int(value)
    else:
        value = float(value)
        if value != value or value in (float("inf"), float("-inf")):
            raise ValueError(f"{section}.{key} must be finite")
    lo, hi = _RANGES.get(key, (None, None))
    if (lo is not None and value < lo) or (hi is not None and value > hi):
        raise ValueError(f"{section}.{key} = {value} is out of range")
    return value


def make_profile(chat: Mapping[str, Any] | None = None, source: str = "", *, duplex: Mapping[str, Any] | None = None,
                 tts: Mapping[str, Any] | None = None) -> dict[str, Any]:
    raw: dict[str, Any] = {"schema": SCHEMA, "version": VERSION, "provenance": {"source": source}}
    for name, section in (("chat", chat), ("duplex", duplex), ("tts", tts)):
        if section:
            raw[name] = dict(section)
    return validate(raw)


def validate(profile: Mapping[str, Any]) -> dict[str, Any]:
    if not isinstance(profile, Mapping) or profile.get("schema") != SCHEMA or profile.get("version") != VERSION:
        raise ValueError("not a runtime.sampling.v1 profile")
    unknown = set(profile) - {"schema", "version", "provenance", *_FIELDS}
    if unknown:
        raise ValueError(f"unknown profile entries: {sorted(unknown)}")
    out: dict[str, Any] = {"schema": SCHEMA, "version": VERSION}
    for section, fields in _FIELDS.items():
        if section not in profile:
            continue
        body = profile[section]
        if not isinstance(body, Mapping):
            raise ValueError(f"{section} must be an object")
        stray = set(body) - set(fields)
        if stray:
            raise ValueError(f"unknown sampling keys: {sorted(stray)}")
        out[section] = {k: _typed(section, k, v) for k, v in body.items()}
    prov = profile.get("provenance", {})
    if not isinstance(prov, Mapping):
        raise ValueError("provenance must be an object")
    out["provenance"] = dict(prov)
    out.setdefault("chat", {})
    return out


def merge_profiles(*profiles: Mapping[str, Any] | None) -> dict[str, Any] | None:
    """Later profiles override earlier ones key by key; the provenance of the last one that says anything wins."""
    out: dict[str, Any] = {"schema": SCHEMA, "version": VERSION}
    used = False
    for raw in profiles:
        if raw is None:
            continue
        prof = validate(raw)
        for section in _FIELDS:
            if prof.get(section):
                out.setdefault(section, {}).update(prof[section])
                used = True
        if prof.get("provenance"):
            out["provenance"] = prof["provenance"]
    if not used:
        return None
    out.setdefault("chat", {})
    out.setdefault("provenance", {})
    return out


def _identity(value: object) -> str:
    return re.sub(r"[^a-z0-9]+", "_", str(value).lower()).strip("_")


def registry_profile(*identities: object) -> dict[str, Any] | None:
    """The registry entry whose key occurs in one of the names (``model_type``, ``architectures``, a path): the longest
    matching key wins, punctuation and case do not matter (``Qwen3NextForCausalLM`` finds ``qwen3_next``)."""
    names = [_identity(v) for v in identities if v]
    for key in sorted(_REGISTRY, key=lambda k: -len(k.replace("_", ""))):
        compact = key.replace("_", "")
        if any(key in n or compact in n.replace("_", "") for n in names):
            return make_profile(_REGISTRY[key], f"architecture-registry:{key}")
    return None


def sidecar_paths(mfq_path) -> tuple[Path, ...]:
    """Where an operator may put overrides: ``<family>.runtime.json`` for a shard ``family-0000i-of-0000N.mfq`` (or
    ``<stem>.runtime.json``), then ``<file>.runtime.json``; the later one overrides the earlier."""
    path = Path(mfq_path)
    exact = Path(f"{path}.runtime.json")
    m = re.match(r"^(.*)-[0-9]{5}-of-[0-9]{5}\.mfq$", path.name)
    family = path.with_name(f"{m.group(1)}.runtime.json") if m else path.with_suffix(".runtime.json")
    return (family, exact) if family != exact else (exact,)


def load_profile(path) -> dict[str, Any]:
    return validate(json.loads(Path(path).read_text(encoding="utf-8")))


def load_sidecar(mfq_path) -> dict[str, Any] | None:
    found = [load_profile(p) for p in sidecar_paths(mfq_path) if p.is_file()]
    return merge_profiles(*found) if found else None


def profile_for_new_checkpoint(source, hf_config: Mapping[str, Any] | None = None, *, assets: Mapping[str, bytes] | None = None,
                               explicit=None, inherited: Mapping[str, Any] | None = None) -> dict[str, Any] | None:
    """The profile to embed in a checkpoint being written, or None when no source says anything."""
    cfg = hf_config or {}
    found = merge_profiles(registry_profile(cfg.get("_name_or_path"), cfg.get("model_type"), *(cfg.get("architectures") or ())),
                           inherited)
    root = Path(source) if source else None
    gen = (assets or {}).get("hf/generation_config.json")
    if gen is None and root is not None and root.is_dir() and (root / "generation_config.json").is_file():
        gen = (root / "generation_config.json").read_bytes()
    if gen is not None:
        found = merge_profiles(found, from_generation_config(gen))
    if root is not None and root.is_dir() and (root / "mfq-runtime.json").is_file():
        found = merge_profiles(found, load_profile(root / "mfq-runtime.json"))
    if explicit:
        found = merge_profiles(found, load_profile(explicit))
    return found


def from_generation_config(text: str | bytes) -> dict[str, Any] | None:
    """Profile from a Hugging Face ``generation_config.json`` (only the keys it actually sets)."""
    cfg = json.loads(text)
    if not isinstance(cfg, Mapping):
        raise ValueError("generation_config.json must be a JSON object")
    if cfg.get("do_sample") is False:
        return make_profile({"temperature": 0.0}, "hf-generation-config")
    names = {"max_new_tokens": "max_tokens", "temperature": "temperature", "top_k": "top_k", "top_p": "top_p",
             "presence_penalty": "presence_penalty", "frequency_penalty": "frequency_penalty", "repetition_penalty": "repetition_penalty"}
    chat = {ours: cfg[theirs] for theirs, ours in names.items() if cfg.get(theirs) is not None}
    return make_profile(chat, "hf-generation-config") if chat else None


def resolve(header_extra: Mapping[str, Any] | None = None, assets: Mapping[str, bytes] | None = None,
            architecture: str | None = None, path=None) -> dict[str, Any]:
    """Effective chat defaults + where they came from (``path``: the checkpoint file, for its sidecars)."""
    out, source = dict(BUILTIN), "builtin"
    reg = registry_profile(architecture) if architecture else None
    if reg is not None:
        out.update(reg["chat"])
        source = reg["provenance"]["source"]
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
    side = load_sidecar(path) if path else None
    if side is not None:
        out.update(side["chat"])
        source = "sidecar"
    return {"chat": out, "source": source}


def merge_request(defaults: Mapping[str, Any], request: Mapping[str, Any]) -> dict[str, Any]:
    """Request values win; ``None`` means "not given"."""
    out = dict(defaults)
    out.update({k: v for k, v in request.items() if v is not None and k in _FIELDS["chat"]})
    return out


def checkpoint_defaults(meta: Mapping[str, Any] | None) -> dict[str, Any]:
    """The chat defaults a checkpoint itself brings (its generation config, its embedded profile, its sidecars -- not
    the registry's guess, not the built-ins): what a server puts under a request that leaves those keys out."""
    meta = meta or {}
    out: dict[str, Any] = {}
    gen = (meta.get("assets") or {}).get("hf/generation_config.json")
    if gen:
        prof = from_generation_config(gen)
        if prof:
            out.update(prof["chat"])
    embedded = (meta.get("header_extra") or {}).get(HEADER_KEY)
    if embedded:
        out.update(validate(embedded)["chat"])
    side = load_sidecar(meta["path"]) if meta.get("path") else None
    if side is not None:
        out.update(side["chat"])
    return out
