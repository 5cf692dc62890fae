"""Reference-logits files (``_logit3_``): baseline log-probabilities of evaluation windows in 16 bits per entry.

A baseline model is run once over ``chunks`` token windows of ``context`` tokens; for the scored second half of each
window (positions ``context // 2 + 1 ..``) the file keeps the full next-token distribution, so any quantized model can
later be scored against it (KL divergence, top-1 agreement, perplexity) without the baseline weights.

Layout (little endian)::

    "_logit3_"  u32 vocab  u32 chunks   chunks x (u32 context, u32 start, u32 count)
    i32 tokens[chunks][context]   f32 target_logp[chunks][count]
    u16 rows[chunks][count][2 * ceil(vocab / 2) + 4]

A row starts with two fp32 (scale = 16 / 65535, offset = log p_max - 16, stored as four u16) followed by one code per
vocabulary entry: ``code = round((logit - max + 16) * 65535 / 16)`` clipped to 16 bits, i.e. log-probabilities down to
16 nats below the maximum at 2.4e-4 resolution.  Byte layout and rounding follow ``mfq/evaluation/reference.py:22-98``.
"""

from __future__ import annotations

import struct
from dataclasses import dataclass
from pathlib import Path
from typing import Callable

import numpy as np

MAGIC = b"_logit3_"
_RANGE = 16.0


def scored_span(context: int) -> tuple[int, int]:
    start = context // 2 + 1
    return start, context - start


def encode_rows(logits: np.ndarray, targets: np.ndarray) -> tuple[np.ndarray, np.ndarray]:
    """``logits [rows, vocab]`` + target ids -> (u16 rows ``[rows, elements]``, fp32 target log-probs)."""
    v = np.asarray(logits, dtype=np.float32)
    vocab = v.shape[1]
    elements = 2 * ((vocab + 1) // 2) + 4
    peak = v.max(-1)
    shifted = v - peak[:, None]
    log_den = np.log(np.exp(shifted).sum(-1))
    target_logp = shifted[np.arange(len(v)), targets] - log_den
    rows = np.zeros((len(v), elements), dtype="<u2")
    head = np.stack((np.full(len(v), _RANGE / 65535, dtype="<f4"), (-log_den).astype("<f4") - np.float32(_RANGE)), axis=-1)
    rows[:, :4] = head.view("<u2").reshape(len(v), 4)
    rows[:, 4 : 4 + vocab] = np.floor((shifted + _RANGE) * (65535 / _RANGE) + 0.5).clip(0, 65535).astype("<u2")
    return rows, target_logp.astype("<f4")


def decode_rows(rows: np.ndarray, vocab: int) -> np.ndarray:
    """u16 rows -> fp32 log-probabilities ``[rows, vocab]``."""
    head = np.ascontiguousarray(rows[:, :4]).view("<f4")  # [rows, 2]: scale, offset
    return rows[:, 4 : 4 + vocab].astype(np.float32) * head[:, :1] + head[:, 1:2]


def write_reference(path, tokens: np.ndarray, logits_fn: Callable[[np.ndarray], np.ndarray]) -> float:
    """``tokens [chunks, context]``; ``logits_fn(window ids) -> [context, vocab]`` logits.  Returns the baseline
    negative log-likelihood summed over all scored positions."""
    tokens = np.asarray(tokens, dtype="<i4")
    chunks, context = tokens.shape
    start, count = scored_span(context)
    if count < 1:
        raise ValueError("windows are too short to score")
    all_rows, all_targets, vocab, nll = [], [], None, 0.0
    for c in range(chunks):
        logits = np.asarray(logits_fn(tokens[c]), dtype=np.float32)
        vocab = logits.shape[1] if vocab is None else vocab
        # the distribution at position i predicts token i + 1: rows start - 1 .. context - 2 score tokens start .. context - 1
        rows, tlp = encode_rows(logits[start - 1 : context - 1], tokens[c, start:])
        all_rows.append(rows)
        all_targets.append(tlp)
        nll -= float(tlp.sum(dtype=np.float64))
    path = Path(path)
    tmp = path.with_name(path.name + ".partial")
    with open(tmp, "wb") as f:
        f.write(MAGIC + struct.pack("<II", vocab, chunks))
        for _ in range(chunks):
            f.write(struct.pack("<III", context, start, count))
        f.write(tokens.tobytes())
        f.write(np.stack(all_targets).astype("<f4").tobytes())
        f.write(np.stack(all_rows).tobytes())
    tmp.replace(path)
    return nll


@dataclass
class Reference:
    vocab: int
    tokens: np.ndarray  # [chunks, context]
    start: int
    count: int
    target_logp: np.ndarray  # [chunks, count]
    rows: np.ndarray  # [chunks, count, elements] u16 (memory mapped)

    def logp(self, chunk: int) -> np.ndarray:
        return decode_rows(np.asarray(self.rows[chunk]), self.vocab)


def read_reference(path) -> Reference:
    raw = np.memmap(path, mode="r", dtype=np.uint8)
    if bytes(raw[:8]) != MAGIC:
        raise ValueError("not a _logit3_ reference file")
    vocab, chunks = struct.unpack_from("<II", raw, 8)
    geo = [struct.unpack_from("<III", raw, 16 + 12 * i) for i in range(chunks)]
    context, start, count = geo[0]
    if any(g != geo[0] for g in geo):
        raise ValueError("windows of different geometry are not supported")
    off = 16 + 12 * chunks
    tokens = np.frombuffer(raw, dtype="<i4", count=chunks * context, offset=off).reshape(chunks, context)
    off += chunks * context * 4
    targets = np.frombuffer(raw, dtype="<f4", count=chunks * count, offset=off).reshape(chunks, count)
    off += chunks * count * 4
    elements = 2 * ((vocab + 1) // 2) + 4
    rows = np.frombuffer(raw, dtype="<u2", count=chunks * count * elements, offset=off).reshape(chunks, count, elements)
    return Reference(vocab, tokens, start, count, targets, rows)


def score_against_reference(path, logits_fn: Callable[[np.ndarray], np.ndarray]) -> dict:
    """KL(baseline || model), top-1 agreement and perplexities of ``logits_fn`` over the windows of a reference file."""
    ref = read_reference(path)
    kl, same, nll, nll_ref, n = 0.0, 0, 0.0, 0.0, 0
    for c in range(ref.tokens.shape[0]):
        ids = ref.tokens[c]
        logits = np.asarray(logits_fn(ids), dtype=np.float32)[ref.start - 1 : len(ids) - 1]
        lq = logits - logits.max(-1, keepdims=True)
        lq = lq - np.log(np.exp(lq).sum(-1, keepdims=True))
        lp = ref.logp(c)
        p = np.exp(lp)
        kl += float((p * (lp - lq)).sum(dtype=np.float64))
        same += int((lp.argmax(-1) == lq.argmax(-1)).sum())
        tgt = ids[ref.start :]
        nll -= float(lq[np.arange(len(tgt)), tgt].sum(dtype=np.float64))
        nll_ref -= float(ref.target_logp[c].sum(dtype=np.float64))
        n += len(tgt)
    return {"kld": kl / n, "same_top": same / n, "ppl": float(np.exp(nll / n)), "ppl_reference": float(np.exp(nll_ref / n)), "tokens": n}
