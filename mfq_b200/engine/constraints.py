"""Token constraints: structured output by masking the logits before sampling.

``response_format = {"type": "json_object"}`` (or ``json_schema``, which is held to "a JSON object") makes the engine
keep a grammar state per row.  Before every step the state's allowed-token mask (computed natively over a byte trie of
the vocabulary, ``native/src/json_constraint.cpp``) becomes an additive bias row -- 0 for allowed tokens, a large
negative number for the others -- that is added to the row's logits ahead of the sampler, inside the captured graph of
the constrained variant of the step; after the step the sampled token advances the state.  The end-of-sequence tokens
are allowed exactly when the document is complete, so a constrained request stops by itself on valid JSON.

Reference: engine token constraints + the tokenizer's grammar (``cpp_runtime/engine/include``: token constraints;
``cpp_runtime/components/tokenizer``: grammar), and ``response_format`` in the OpenAI-compatible request parser
(``mfq/server/api/openai_compat.py:125``).
"""

from __future__ import annotations

import numpy as np
import torch

NEG = -1.0e30  # representable in bf16; exp() of it is 0 and an arg-max never picks it


class JsonTokenConstraint:
    def __init__(self, vocabulary, stop_ids, need_object: bool = True) -> None:
        from .. import native
        self.vocabulary = vocabulary
        self.stop_ids = tuple(int(t) for t in stop_ids if t is not None and 0 <= int(t) < vocabulary.size)
        self.state = native.JsonState(vocabulary, need_object)
        self.finished = False

    def allowed(self) -> np.ndarray:
        mask = self.state.mask()
        if self.state.complete or not mask.any():  # complete, or a dead end (depth limit): let the request end
            mask[list(self.stop_ids)] = True
        return mask

    def bias(self, width: int) -> torch.Tensor:
        """bf16 ``[width]``: 0 where a token may come next, a large negative number elsewhere (ids past the
        vocabulary, e.g. padding columns of the output projection, are never allowed)."""
        cache = self.vocabulary.__dict__.setdefault("_bias_cache", {})
        key = (self.state.key, self.state.complete, self.stop_ids, width)
        hit = cache.get(key)
        if hit is not None:  # e.g. every step inside a string value: same state, same 256 KB row
            return hit
        out = np.full(width, NEG, dtype=np.float32)
        mask = self.allowed()
        n = min(width, mask.size)
        out[:n][mask[:n]] = 0.0
        row = torch.from_numpy(out).to(torch.bfloat16)
        if len(cache) >= 128:
            cache.pop(next(iter(cache)))
        cache[key] = row
        return row

    def advance(self, token: int) -> None:
        if self.finished:
            return
        if token in self.stop_ids or not self.state.feed_token(int(token)):
            self.finished = True


class LogitBias:
    """OpenAI ``logit_bias``: a fixed additive bias on chosen token ids for the whole request (values are clamped to
    +-100 as the API defines them); optionally on top of a grammar constraint."""

    def __init__(self, bias: dict, inner=None) -> None:
        self.table = {int(t): max(-100.0, min(100.0, float(v))) for t, v in bias.items()}
        self.inner = inner
        self.finished = False

    def bias(self, width: int) -> torch.Tensor:
        out = self.inner.bias(width).float() if self.inner is not None else torch.zeros(width)
        for t, v in self.table.items():
            if 0 <= t < width:
                out[t] += v
        return out.to(torch.bfloat16)

    def advance(self, token: int) -> None:
        if self.inner is not None:
            self.inner.advance(token)
            self.finished = self.inner.finished


def make_constraint(response_format, vocabulary, stop_ids):
    """``response_format`` as the request carried it (a dict, a type string or None) -> a constraint or None."""
    if not response_format or vocabulary is None:
        return None
    kind = response_format.get("type") if isinstance(response_format, dict) else str(response_format)
    if kind in ("json_object", "json_schema", "json"):
        return JsonTokenConstraint(vocabulary, stop_ids, need_object=True)
    return None
