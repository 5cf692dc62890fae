"""API keys with scopes.

Three scopes: ``inference`` (the OpenAI / Anthropic routes), ``read`` (GET on the control API, metrics), ``admin``
(everything, including changing the server: loading models, jobs, cache purges, key management).  Keys are kept as
SHA-256 digests, so the store can be written to disk and listed without revealing a key; a key is shown once, when it is
created.  Whether credentials are enforced is decided once, when the store is made: a store that was given a key or a
key file enforces them from then on, also when its table later becomes empty (every request is then refused, and the
last admin key cannot be revoked); a store made with neither leaves the server open (the default for a loopback
deployment).  Reference:
``mfq/server/api/auth.py`` (bearer / ``x-api-key`` credentials with scopes) and the auth-key routes of the control API.
"""

from __future__ import annotations

import hashlib
import hmac
import json
import secrets
import time
from pathlib import Path

SCOPES = ("inference", "read", "admin")
_OPEN_PATHS = ("/health", "/health/identity")


def required_scope(method: str, path: str) -> str | None:
    """Scope a request needs (None: no credential needed)."""
    if path in _OPEN_PATHS:
        return None
    if path.startswith("/v1"):
        return "read" if method == "GET" else "inference"
    if path.startswith("/api/v1/auth"):
        return "admin"
    if path.startswith("/api/v1/evaluations/"):
        return "inference"  # runs the model on caller text, changes nothing
    if method in ("GET", "HEAD", "OPTIONS"):
        return "read"
    return "admin"


def _digest(key: str) -> str:
    return hashlib.sha256(key.encode()).hexdigest()


class KeyStore:
    def __init__(self, path=None, enforce: bool | None = None) -> None:
        self.path = Path(path) if path else None
        self.keys: dict[str, dict] = {}  # digest -> {"id", "name", "scopes", "created"}
        if self.path and self.path.exists():
            self.keys = json.loads(self.path.read_text())
        # auth on or off is a property of the deployment, not of how many keys happen to be in the table
        self.enforce = bool(self.path is not None or self.keys) if enforce is None else bool(enforce)

    def _save(self) -> None:
        if self.path:
            tmp = self.path.with_suffix(".tmp")
            tmp.write_text(json.dumps(self.keys, indent=1))
            tmp.replace(self.path)

    def add(self, key: str, scopes=("admin",), name: str = "") -> dict:
        scopes = [s for s in SCOPES if s in scopes]
        if not scopes:
            raise ValueError(f"a key needs at least one scope of {SCOPES}")
        rec = {"id": secrets.token_hex(6), "name": name, "scopes": scopes, "created": time.time()}
        self.keys[_digest(key)] = rec
        self.enforce = True
        self._save()
        return rec

    def create(self, scopes=("inference",), name: str = "") -> tuple[str, dict]:
        key = "mfq-" + secrets.token_urlsafe(32)
        return key, self.add(key, scopes, name)

    def revoke(self, key_id: str) -> bool:
        """Remove a key.  The last key with the ``admin`` scope stays (ValueError): without it nobody could manage keys."""
        for d, rec in list(self.keys.items()):
            if rec["id"] == key_id:
                if "admin" in rec["scopes"] and sum("admin" in r["scopes"] for r in self.keys.values()) == 1:
                    raise ValueError("the last admin key cannot be revoked")
                del self.keys[d]
                self._save()
                return True
        return False

    def listing(self) -> list[dict]:
        return sorted(self.keys.values(), key=lambda r: r["created"])

    def scopes_of(self, key: str | None) -> list[str] | None:
        if not key:
            return None
        want = _digest(key)
        for d, rec in self.keys.items():
            if hmac.compare_digest(d, want):
                return rec["scopes"]
        return None

    def allows(self, key: str | None, scope: str | None) -> bool:
        if scope is None or not self.enforce:
            return True
        have = self.scopes_of(key)
        return have is not None and ("admin" in have or scope in have)
