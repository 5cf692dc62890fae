"""Speculative-decoding policies: how a draft chain is verified and how deep the next chain should be.

* :func:`verify_greedy` -- the longest prefix of the draft that equals the target's arg-max tokens, plus the target's own
  token after it (what the engine's device-side accept kernel computes).
* :func:`verify_stochastic` -- speculative sampling: draft token ``x`` with draft probability ``q(x)`` is kept with
  probability ``min(1, p(x) / q(x))``; at the first rejection the replacement is drawn from ``max(0, p - q)``
  renormalised, and if every draft survives one more token is drawn from the target's next distribution.  The emitted
  tokens are distributed exactly as if the target had been sampled alone.
* :class:`DepthController` -- keeps an exponential average of the acceptance at every draft position and of the measured
  cycle time at every depth, scores a depth by expected tokens per millisecond, explores unmeasured depths first,
  re-probes stale ones, and parks speculation (depth 0) only when the best speculative score falls below the plain
  decode score by a margin.

Reference: ``cpp_runtime/engine/include/mtp_policy.h`` (greedy / stochastic / compact-top-k chain verification) and
``mtp_depth_controller.h`` (adaptive depth, parking).
"""

from __future__ import annotations

import torch


def verify_greedy(draft: torch.Tensor, target_argmax: torch.Tensor) -> tuple[int, int]:
    """``draft [K]`` tokens, ``target_argmax [K + 1]`` = the target's choice after each prefix.  Returns (number of
    accepted drafts, the token that follows them)."""
    k = int(draft.numel())
    same = (draft.to(torch.int64) == target_argmax[:k].to(torch.int64)).to(torch.int64)
    n = int(same.cumprod(0).sum())
    return n, int(target_argmax[n])


def verify_stochastic(draft: torch.Tensor, draft_probs: torch.Tensor, target_probs: torch.Tensor,
                      generator: torch.Generator | None = None) -> tuple[int, int]:
    """``draft [K]``, ``draft_probs [K, V]`` (the distributions the drafts were sampled from), ``target_probs [K + 1, V]``.
    Returns (accepted drafts, next token)."""
    k = int(draft.numel())
    u = torch.rand(k, generator=generator)
    for i in range(k):
        x = int(draft[i])
        p, q = float(target_probs[i, x]), float(draft_probs[i, x])
        if q > 0 and float(u[i]) < min(1.0, p / q):
            continue
        residual = (target_probs[i] - draft_probs[i]).clamp_min(0)
        total = float(residual.sum())
        dist = residual / total if total > 0 else target_probs[i]
        return i, int(torch.multinomial(dist, 1, generator=generator))
    return k, int(torch.multinomial(target_probs[k], 1, generator=generator))


class DepthController:
    def __init__(self, max_depth: int = 3, *, ema: float = 0.2, exit_margin: float = 1.15, reprobe_every: int = 64,
                 park_after: int = 8) -> None:
        self.max_depth = max(1, int(max_depth))
        self.ema, self.exit_margin, self.reprobe_every, self.park_after = ema, exit_margin, reprobe_every, park_after
        self.acceptance = [0.6] + [0.5] * (self.max_depth - 1)  # P(draft i accepted | drafts before it accepted)
        self.cycle_ms: list[float | None] = [None] * (self.max_depth + 1)  # index = depth, 0 = plain decode
        self.age = [0] * (self.max_depth + 1)  # cycles since the depth was last measured
        self.losing_streak = 0
        self.parked = False

    # ---- model of a cycle ------------------------------------------------------------------------------------------
    def expected_tokens(self, depth: int) -> float:
        total, alive = 1.0, 1.0
        for i in range(depth):
            alive *= self.acceptance[i]
            total += alive
        return total

    def score(self, depth: int) -> float | None:
        ms = self.cycle_ms[depth]
        return None if ms is None or ms <= 0 else self.expected_tokens(depth) / ms

    # ---- decisions --------------------------------------------------------------------------------------------------
    def next_depth(self) -> int:
        for d in [0] + list(range(self.max_depth, 0, -1)):  # measure plain decode, then every depth, widest first
            if self.cycle_ms[d] is None:
                return d
        stale = max(range(self.max_depth + 1), key=lambda d: self.age[d])
        if self.age[stale] >= self.reprobe_every:
            return stale
        if self.parked:
            return 0
        return max(range(1, self.max_depth + 1), key=lambda d: self.score(d) or 0.0)

    def observe(self, depth: int, accepted: int, cycle_ms: float) -> None:
        depth = min(max(depth, 0), self.max_depth)
        accepted = min(max(accepted, 0), depth)
        for i in range(depth):
            if i <= accepted:  # position i was reached; it was accepted iff i < accepted
                hit = 1.0 if i < accepted else 0.0
                self.acceptance[i] += self.ema * (hit - self.acceptance[i])
        old = self.cycle_ms[depth]
        self.cycle_ms[depth] = cycle_ms if old is None else old + self.ema * (cycle_ms - old)
        for d in range(self.max_depth + 1):
            self.age[d] = 0 if d == depth else self.age[d] + 1
        base = self.score(0)
        best = max((self.score(d) or 0.0) for d in range(1, self.max_depth + 1))
        if base is not None and all(self.cycle_ms[d] is not None for d in range(1, self.max_depth + 1)):
            if best < base * self.exit_margin:
                self.losing_streak += 1
            else:
                self.losing_streak = 0
                self.parked = False
            if self.losing_streak >= self.park_after:
                self.parked = True

    def state(self) -> dict:
        return {"acceptance": [round(a, 3) for a in self.acceptance], "cycle_ms": self.cycle_ms, "parked": self.parked,
                "expected_tokens": [round(self.expected_tokens(d), 3) for d in range(self.max_depth + 1)]}


class CycleDepthController(DepthController):
    """Depth choice among draft/verify cycles only (depths 1 .. max): what the engine uses when parking is off or is
    decided elsewhere (:class:`ParkingController`).  Plain decoding (depth 0) is never probed or chosen."""

    def next_depth(self) -> int:
        for d in range(self.max_depth, 0, -1):  # measure every depth once, widest first
            if self.cycle_ms[d] is None:
                return d
        stale = max(range(1, self.max_depth + 1), key=lambda d: self.age[d])
        if self.age[stale] >= self.reprobe_every:
            return stale
        return max(range(1, self.max_depth + 1), key=lambda d: self.score(d) or 0.0)


class ParkingController:
    """Run draft/verify cycles only while they pay: the engine-side reduction of :class:`DepthController` to the two
    modes one captured graph geometry offers -- cycles at the depth the engine was built with, or plain decode steps
    that keep the draft head primed ("parked").

    Both modes are measured in tokens per row and millisecond (EMA).  After ``probe`` calls in each mode the controller
    parks when cycles have been slower than ``exit_margin`` x plain decoding for ``park_after`` calls in a row, re-probes
    cycles for ``probe`` calls every ``reprobe_every`` parked calls, and resumes when they win again.  Reference:
    ``cpp_runtime/engine/include/mtp_depth_controller.h`` (adaptive depth with parking)."""

    def __init__(self, *, ema: float = 0.2, exit_margin: float = 1.05, park_after: int = 8, reprobe_every: int = 64,
                 probe: int = 4) -> None:
        self.ema, self.exit_margin, self.park_after, self.reprobe_every, self.probe = ema, exit_margin, park_after, reprobe_every, probe
        self.rate = {"mtp": None, "plain": None}  # tokens per row per ms
        self.calls = {"mtp": 0, "plain": 0}
        self.parked = False
        self.losing = 0
        self._parked_calls = 0
        self._probe_left = 0

    def mode(self) -> str:
        if self.calls["mtp"] < self.probe:
            return "mtp"
        if self.calls["plain"] < self.probe:
            return "plain"
        if self.parked:
            if self._probe_left > 0:
                return "mtp"
            if self._parked_calls >= self.reprobe_every:
                self._probe_left = self.probe
                self._parked_calls = 0
                return "mtp"
            return "plain"
        return "mtp"

    def observe(self, mode: str, tokens: int, rows: int, ms: float) -> None:
        if rows <= 0 or ms <= 0:
            return
        r = tokens / rows / ms
        old = self.rate[mode]
        self.rate[mode] = r if old is None else old + self.ema * (r - old)
        self.calls[mode] += 1
        if self.parked:
            if mode == "plain":
                self._parked_calls += 1
            else:
                self._probe_left -= 1
        if self.rate["mtp"] is None or self.rate["plain"] is None or self.calls["plain"] < self.probe:
            return
        wins = self.rate["mtp"] >= self.rate["plain"] * self.exit_margin
        if self.parked:
            if mode == "mtp" and self._probe_left <= 0 and wins:
                self.parked, self.losing = False, 0
        elif mode == "mtp":
            self.losing = 0 if wins else self.losing + 1
            if self.losing >= self.park_after:
                self.parked, self._parked_calls, self._probe_left = True, 0, 0

    def state(self) -> dict:
        return {"parked": self.parked, "rate": dict(self.rate), "calls": dict(self.calls), "losing": self.losing}
