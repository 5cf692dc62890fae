"""Per-model policies that outlive the server process.

An operator sets them over REST (``PUT /api/v1/runtime/policies/{model}``), they are kept in a JSON file beside the
server's other state and applied to every later request for that model:

* ``inference``: request defaults (``temperature``, ``top_p``, ``top_k``, ``max_tokens``, ``enable_mtp``, ...) used for
  the fields a request leaves out -- a request's own value always wins;
* ``concurrency``: ``max_queue`` and ``queue_timeout`` of the model's scheduler, applied at once and at every load;
* ``context`` (``max_context_tokens``) and ``memory`` (``kv_budget_gb``, ``moe_gpu_cache_gb``): read by the loader the
  next time the model is loaded.

Reference: the control API keeps context / memory / concurrency / inference policies per model
(``mfq/server/api/routes/runtime.py``, ``docs/cli/serve.md``: "per-model persisted policies").
"""

from __future__ import annotations

import json
import os
import threading
from pathlib import Path

SECTIONS = {
    "inference": {"temperature": float, "top_p": float, "top_k": int, "max_tokens": int, "presence_penalty": float,
                  "frequency_penalty": float, "repetition_penalty": float, "enable_mtp": bool, "mtp_max_draft_tokens": int},
    "concurrency": {"max_queue": int, "queue_timeout": float},
    "context": {"max_context_tokens": int},
    "memory": {"kv_budget_gb": float, "moe_gpu_cache_gb": float},
}


def validate(doc: dict) -> dict:
    out: dict = {}
    for section, values in (doc or {}).items():
        if section not in SECTIONS:
            raise ValueError(f"unknown policy section {section!r}; known: {', '.join(SECTIONS)}")
        if not isinstance(values, dict):
            raise ValueError(f"policy section {section!r} must be an object")
        clean = {}
        for key, value in values.items():
            kind = SECTIONS[section].get(key)
            if kind is None:
                raise ValueError(f"unknown key {key!r} in policy section {section!r}")
            if kind is bool:
                if not isinstance(value, bool):
                    raise ValueError(f"{section}.{key} must be true or false")
                clean[key] = value
            else:
                if isinstance(value, bool) or not isinstance(value, (int, float)):
                    raise ValueError(f"{section}.{key} must be a number")
                if value < 0:
                    raise ValueError(f"{section}.{key} must not be negative")
                clean[key] = kind(value)
        out[section] = clean
    return out


class PolicyStore:
    def __init__(self, path=None) -> None:
        self.path = Path(path) if path else None
        self._lock = threading.Lock()
        self._doc: dict[str, dict] = {}
        if self.path and self.path.exists():
            try:
                self._doc = {m: validate(p) for m, p in json.loads(self.path.read_text()).items()}
            except (OSError, ValueError):
                self._doc = {}

    def all(self) -> dict:
        with self._lock:
            return json.loads(json.dumps(self._doc))

    def get(self, model: str) -> dict:
        with self._lock:
            return json.loads(json.dumps(self._doc.get(model, {})))

    def put(self, model: str, doc: dict) -> dict:
        clean = validate(doc)
        with self._lock:
            if clean:
                self._doc[model] = clean
            else:
                self._doc.pop(model, None)
            self._save()
        return clean

    def _save(self) -> None:
        if not self.path:
            return
        self.path.parent.mkdir(parents=True, exist_ok=True)
        tmp = self.path.with_name(self.path.name + f".tmp-{os.getpid()}")
        tmp.write_text(json.dumps(self._doc, indent=1))
        os.replace(tmp, self.path)

    # ---- application -------------------------------------------------------------------------------------------------
    def request_defaults(self, model: str, body: dict) -> dict:
        """``body`` with the model's inference defaults filled into the fields it leaves out."""
        defaults = self.get(model).get("inference", {})
        if not defaults:
            return body
        merged = dict(body)
        for key, value in defaults.items():
            if key == "max_tokens" and (body.get("max_tokens") or body.get("max_completion_tokens")):
                continue
            if body.get(key) is None:
                merged[key] = value
        return merged

    def apply_concurrency(self, model: str, scheduler) -> None:
        c = self.get(model).get("concurrency", {})
        if "max_queue" in c:
            scheduler.max_queue = c["max_queue"]
        if "queue_timeout" in c and hasattr(scheduler, "queue_timeout"):
            scheduler.queue_timeout = c["queue_timeout"] or None
