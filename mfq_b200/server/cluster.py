"""Cluster backend: route a model name to one of several remote servers of this kind.

Every peer is polled (``GET /health``, ``GET /v1/models``); a request for a model that is not loaded locally is sent
to a healthy peer that lists it -- the least recently used one among them, so load spreads -- and a peer that fails a
request or a poll is taken out of rotation for ``cooldown`` seconds before it is probed again.  The transport is a
callable ``fetch(method, url, json_body, headers, stream) -> (status, body | line iterator)`` so tests run without a
network; the default uses ``requests``.  Reference: ``mfq/server/runtime/cluster.py`` (health-aware routing of a model
name to remote MFQ servers).
"""

from __future__ import annotations

import json
import threading
import time
from dataclasses import dataclass, field


def _requests_fetch(method: str, url: str, body, headers: dict, stream: bool, timeout: float = 600.0):
    import requests
    r = requests.request(method, url, json=body, headers=headers, stream=stream, timeout=timeout)
    if stream:
        return r.status_code, (line + b"\n" for line in r.iter_lines())
    try:
        return r.status_code, r.json()
    except ValueError:
        return r.status_code, {"raw": r.text}


@dataclass
class Peer:
    url: str
    api_key: str | None = None
    models: list[str] = field(default_factory=list)
    healthy: bool = False
    last_poll: float = 0.0
    down_until: float = 0.0
    last_used: float = 0.0
    failures: int = 0

    def headers(self) -> dict:
        return {"authorization": f"Bearer {self.api_key}"} if self.api_key else {}


class NoPeer(Exception):
    """No healthy peer serves the model."""


class ClusterBackend:
    def __init__(self, peers: list[str | dict], *, fetch=None, poll_interval: float = 5.0, cooldown: float = 15.0,
                 clock=time.monotonic) -> None:
        self.peers = [Peer(**p) if isinstance(p, dict) else Peer(p.rstrip("/")) for p in peers]
        self.fetch = fetch or _requests_fetch
        self.poll_interval, self.cooldown, self.clock = poll_interval, cooldown, clock
        self._lock = threading.Lock()
        self._tick = 0

    # ---- health --------------------------------------------------------------------------------------------------
    def _poll(self, peer: Peer) -> None:
        now = self.clock()
        peer.last_poll = now
        try:
            status, health = self.fetch("GET", peer.url + "/health", None, peer.headers(), False)
            ok = status == 200 and isinstance(health, dict) and health.get("status") in ("ok", "degraded")
            if ok:
                status, listing = self.fetch("GET", peer.url + "/v1/models", None, peer.headers(), False)
                ok = status == 200
                if ok:
                    peer.models = [m["id"] for m in listing.get("data", [])]
        except Exception:
            ok = False
        if ok:
            peer.healthy, peer.failures = True, 0
        else:
            self._mark_down(peer)

    def _mark_down(self, peer: Peer) -> None:
        peer.healthy = False
        peer.failures += 1
        peer.down_until = self.clock() + self.cooldown

    def refresh(self, force: bool = False) -> None:
        now = self.clock()
        for peer in self.peers:
            if now < peer.down_until and not force:
                continue
            if force or now - peer.last_poll >= self.poll_interval or not peer.last_poll:
                self._poll(peer)

    # ---- routing -------------------------------------------------------------------------------------------------
    def models(self) -> list[str]:
        self.refresh()
        return sorted({m for p in self.peers if p.healthy for m in p.models})

    def pick(self, model: str) -> Peer:
        with self._lock:
            self.refresh()
            able = [p for p in self.peers if p.healthy and model in p.models]
            if not able:
                raise NoPeer(model)
            peer = min(able, key=lambda p: p.last_used)
            self._tick += 1
            peer.last_used = self._tick  # a counter, not a time stamp: two picks inside one clock tick still alternate
            return peer

    def forward(self, path: str, body: dict, stream: bool = False):
        """Send ``body`` to a peer serving ``body["model"]``; on a transport failure or a 5xx answer the peer leaves the
        rotation and the next one is tried.  Returns (status, json | line iterator, peer url)."""
        tried = 0
        while True:
            peer = self.pick(body.get("model", ""))
            tried += 1
            try:
                status, out = self.fetch("POST", peer.url + path, body, peer.headers(), stream)
            except Exception:
                status, out = 599, None
            if status >= 500:
                with self._lock:
                    self._mark_down(peer)
                if tried < len(self.peers):
                    continue
                if out is None:
                    raise NoPeer(body.get("model", ""))
            return status, out, peer.url

    def status(self) -> list[dict]:
        return [{"url": p.url, "healthy": p.healthy, "models": p.models, "failures": p.failures,
                 "cooling_down": self.clock() < p.down_until} for p in self.peers]
