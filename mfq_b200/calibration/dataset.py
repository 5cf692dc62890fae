"""Calibration corpora: tokenized text or model-generated traces, split into train / validation, packed into windows.

Two builders, both from LOCAL files (JSONL or plain text; nothing is downloaded):

* :func:`build_text_corpus` -- records ``{"text": ...}`` or ``{"messages": [...]}`` (or plain-text files, one record per
  paragraph) grouped into named domains; every domain contributes to both splits in proportion to its weight, records
  are shuffled with a per-domain seed, tokenized, concatenated and packed into windows of ``sequence_length`` tokens.
* :func:`build_trace_corpus` -- JSONL rows written by a generator model (``model``, ``mode`` thinking / nonthinking,
  ``finish_reason`` = stop, ``messages`` ending at a user or tool turn, ``output``, optional ``reasoning``): the rendered
  conversation is one window per record and carries a loss mask that scores only the generated part.

Artifact (a directory): ``manifest.json`` (``format`` ``mfq.calibration-corpus.v1``, or ``.v2`` with a loss mask; seed,
sequence length, domains and weights, target / actual token counts per split, per-split record counts and a SHA-256 over
their hashes, tokenizer identity, sources, ``token_sha256``), ``tokens.npy`` (int32, all windows concatenated),
``offsets.npy`` (int64, window i = ``tokens[offsets[i]:offsets[i+1]]``), ``split_ids.npy`` (uint8: 0 train, 1
validation), ``domain_ids.npy`` (uint16) and, for v2, ``loss_mask.npy`` (uint8, 1 = position is scored).

Reference: ``mfq/calibration/dataset.py`` (``build_corpus_from_records`` :611, ``build_trace_corpus_from_jsonl`` :956,
``_write_corpus_artifact`` :558, ``_trace_record`` :384) -- the artifact layout is the same so either side reads the
other's corpora; the reference's builders additionally fetch their sources from a model hub.
"""

from __future__ import annotations

import hashlib
import json
import os
import shutil
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Iterable, Iterator, Mapping, Sequence

import numpy as np

FORMAT = "mfq.calibration-corpus.v1"
MASKED_FORMAT = "mfq.calibration-corpus.v2"
SPLITS = {"train": 0, "validation": 1}


@dataclass
class CalibrationCorpus:
    root: Path
    manifest: dict[str, Any]
    tokens: np.ndarray
    offsets: np.ndarray
    split_ids: np.ndarray
    domain_ids: np.ndarray
    loss_mask: np.ndarray | None = None

    @property
    def chunks(self) -> int:
        return int(self.offsets.size - 1)

    def chunk_tokens(self, i: int) -> np.ndarray:
        return self.tokens[int(self.offsets[i]) : int(self.offsets[i + 1])]

    def chunk_loss_mask(self, i: int) -> np.ndarray:
        """1 where the token at that position is a prediction target that counts (position 0 never is)."""
        a, b = int(self.offsets[i]), int(self.offsets[i + 1])
        if self.loss_mask is None:
            m = np.ones(b - a, dtype=np.uint8)
            m[0] = 0
            return m
        return self.loss_mask[a:b]

    def token_count(self, split: str | None = None) -> int:
        sizes = np.diff(self.offsets)
        return int(sizes.sum() if split is None else sizes[self.split_ids == SPLITS[split]].sum())

    def iter_chunks(self, split: str, max_tokens: int | None = None) -> Iterator[tuple[np.ndarray, np.ndarray]]:
        """Windows of one split in stored order (tokens, loss mask), until ``max_tokens`` tokens have been yielded."""
        seen = 0
        for i in np.flatnonzero(self.split_ids == SPLITS[split]):
            if max_tokens is not None and seen >= max_tokens:
                return
            t = self.chunk_tokens(int(i))
            seen += t.size
            yield t, self.chunk_loss_mask(int(i))


def load_corpus(path) -> CalibrationCorpus:
    root = Path(path)
    manifest = json.loads((root / "manifest.json").read_text(encoding="utf-8"))
    if manifest.get("format") not in (FORMAT, MASKED_FORMAT):
        raise ValueError(f"{root} is not a calibration corpus (format {manifest.get('format')!r})")
    tokens = np.load(root / "tokens.npy", allow_pickle=False)
    offsets = np.load(root / "offsets.npy", allow_pickle=False)
    mask = np.load(root / "loss_mask.npy", allow_pickle=False) if (root / "loss_mask.npy").exists() else None
    if manifest["format"] == MASKED_FORMAT and mask is None:
        raise ValueError("a v2 corpus needs loss_mask.npy")
    if offsets[-1] != tokens.size or (mask is not None and mask.size != tokens.size):
        raise ValueError("corpus arrays disagree in length")
    digest = hashlib.sha256(np.ascontiguousarray(tokens, dtype="<i4").tobytes()).hexdigest()
    if manifest.get("token_sha256") not in (None, digest):
        raise ValueError("tokens.npy does not match the manifest's token_sha256")
    return CalibrationCorpus(root, manifest, tokens, offsets, np.load(root / "split_ids.npy", allow_pickle=False),
                             np.load(root / "domain_ids.npy", allow_pickle=False), mask)


def pack_stream(tokens: Sequence[int], sequence_length: int) -> list[np.ndarray]:
    """Cut a token stream into windows of ``sequence_length``; no window is shorter than two tokens (a remainder of
    one token is absorbed by shortening the window before it)."""
    if sequence_length < 2:
        raise ValueError("sequence_length must be at least 2")
    n = len(tokens)
    if n < 2:
        raise ValueError("a stream needs at least two tokens")
    out, cur = [], 0
    while cur < n:
        left = n - cur
        take = left if left <= sequence_length else (sequence_length - 1 if left == sequence_length + 1 else sequence_length)
        if sequence_length == 2 and left == 3:
            take = 3
        out.append(np.asarray(tokens[cur : cur + take], dtype=np.int32))
        cur += take
    return out


def _write(output: Path, chunks, split_ids, domain_ids, manifest, loss_masks=None) -> CalibrationCorpus:
    if not chunks:
        raise ValueError("calibration corpus has no windows")
    if output.exists():
        raise FileExistsError(f"calibration corpus already exists: {output}")
    offsets = np.zeros(len(chunks) + 1, dtype=np.int64)
    offsets[1:] = np.cumsum([c.size for c in chunks])
    tokens = np.concatenate(chunks).astype(np.int32, copy=False)
    manifest = dict(manifest)
    manifest["token_sha256"] = hashlib.sha256(np.ascontiguousarray(tokens, dtype="<i4").tobytes()).hexdigest()
    tmp = output.with_name(output.name + ".tmp")
    if tmp.exists():
        shutil.rmtree(tmp)
    tmp.mkdir(parents=True)
    try:
        (tmp / "manifest.json").write_text(json.dumps(manifest, ensure_ascii=False, indent=2), encoding="utf-8")
        np.save(tmp / "tokens.npy", tokens, allow_pickle=False)
        np.save(tmp / "offsets.npy", offsets, allow_pickle=False)
        np.save(tmp / "split_ids.npy", np.asarray(split_ids, dtype=np.uint8), allow_pickle=False)
        np.save(tmp / "domain_ids.npy", np.asarray(domain_ids, dtype=np.uint16), allow_pickle=False)
        if loss_masks is not None:
            np.save(tmp / "loss_mask.npy", np.concatenate(loss_masks).astype(np.uint8, copy=False), allow_pickle=False)
        os.replace(tmp, output)
    except BaseException:
        shutil.rmtree(tmp, ignore_errors=True)
        raise
    return load_corpus(output)


def _file_identity(path: Path) -> dict[str, Any]:
    h = hashlib.sha256()
    with path.open("rb") as f:
        for block in iter(lambda: f.read(1 << 20), b""):
            h.update(block)
    return {"path": str(path), "bytes": path.stat().st_size, "sha256": h.hexdigest()}


def _tokenizer_identity(tokenizer: Any) -> dict[str, Any]:
    vocab = getattr(tokenizer, "vocab_size", None)
    return {"class": type(tokenizer).__name__, "vocab_size": int(vocab) if isinstance(vocab, int) else None,
            "name": str(getattr(tokenizer, "name_or_path", "") or "")}


def _encode(tokenizer: Any, text: str) -> list[int]:
    ids = tokenizer.encode(text)
    return list(ids if not hasattr(ids, "ids") else ids.ids)


def _render(tokenizer: Any, record: Mapping[str, Any], render_mode: str) -> str:
    if "messages" in record and render_mode != "plain":
        return tokenizer.apply_chat_template(list(record["messages"]), add_generation_prompt=False)
    if "messages" in record:
        return "\n".join(str(m.get("content", "")) for m in record["messages"])
    if "text" not in record:
        raise ValueError("a calibration record needs `text` or `messages`")
    return str(record["text"])


def read_records(path) -> list[dict[str, Any]]:
    """JSONL (one object per line) or plain text (paragraphs separated by blank lines)."""
    p = Path(path)
    if p.suffix.lower() in (".jsonl", ".json"):
        rows = [json.loads(line) for line in p.read_text(encoding="utf-8").splitlines() if line.strip()]
        return [r if isinstance(r, dict) else {"text": str(r)} for r in rows]
    return [{"text": para.strip()} for para in p.read_text(encoding="utf-8").split("\n\n") if para.strip()]


def _largest_remainder(total: int, weights: Mapping[str, float]) -> dict[str, int]:
    s = sum(weights.values())
    raw = {k: total * v / s for k, v in weights.items()}
    out = {k: int(v) for k, v in raw.items()}
    for k in sorted(raw, key=lambda k: raw[k] - out[k], reverse=True)[: total - sum(out.values())]:
        out[k] += 1
    return out


def build_text_corpus(tokenizer: Any, output, sources: Mapping[str, Iterable[Mapping[str, Any]]], *, train_tokens: int,
                      validation_tokens: int, sequence_length: int = 2048, seed: int = 0, render_mode: str = "auto",
                      domain_weights: Mapping[str, float] | None = None, source_files: Sequence[Path] = ()) -> CalibrationCorpus:
    """``sources``: domain name -> records.  Every split takes its token quota from every domain (largest-remainder
    shares of ``domain_weights``, equal by default); train and validation never share a record."""
    domains = sorted(sources)
    if not domains:
        raise ValueError("no calibration sources")
    weights = {d: float((domain_weights or {}).get(d, 1.0)) for d in domains}
    quota = {"train": _largest_remainder(train_tokens, weights), "validation": _largest_remainder(validation_tokens, weights)}
    chunks, split_ids, domain_ids = [], [], []
    record_counts = {s: {} for s in SPLITS}
    record_sets = {s: {} for s in SPLITS}
    for di, d in enumerate(domains):
        records = list(sources[d])
        order = np.random.default_rng(int.from_bytes(hashlib.sha256(f"{seed}:{d}".encode()).digest()[:8], "little")).permutation(len(records))
        cursor = 0
        for split in ("validation", "train"):  # validation first: it is small and must not starve
            want = quota[split][d]
            stream, hashes = [], []
            while len(stream) < want and cursor < len(records):
                text = _render(tokenizer, records[int(order[cursor])], render_mode)
                cursor += 1
                ids = _encode(tokenizer, text)
                if not ids:
                    continue
                hashes.append(hashlib.sha256(text.encode("utf-8")).hexdigest())
                stream.extend(ids)
            if want and len(stream) < want:
                raise ValueError(f"domain {d!r} has too few tokens for its {split} quota ({len(stream)} < {want})")
            stream = stream[:want]
            record_counts[split][d] = len(hashes)
            record_sets[split][d] = {"count": len(hashes), "sha256": hashlib.sha256("\n".join(hashes).encode("ascii")).hexdigest()}
            if len(stream) >= 2:
                for c in pack_stream(stream, sequence_length):
                    chunks.append(c)
                    split_ids.append(SPLITS[split])
                    domain_ids.append(di)
    actual = {s: int(sum(c.size for c, k in zip(chunks, split_ids) if k == SPLITS[s])) for s in SPLITS}
    manifest = {"format": FORMAT, "seed": int(seed), "sequence_length": int(sequence_length), "domains": domains,
                "domain_weights": weights, "target_tokens": {"train": int(train_tokens), "validation": int(validation_tokens)},
                "actual_tokens": actual, "record_counts": record_counts, "record_sets": record_sets,
                "tokenizer": {**_tokenizer_identity(tokenizer), "render_mode": render_mode},
                "sources": {"files": [_file_identity(Path(p)) for p in source_files]}}
    return _write(Path(output), chunks, split_ids, domain_ids, manifest)


def trace_record(row: Mapping[str, Any], *, expected_generator_model: str | None = None) -> tuple[list[dict], str, str]:
    """Validate one generated trace; returns (messages including the generated assistant turn, mode, source dataset)."""
    model = str(row.get("model", "")).strip()
    if expected_generator_model and model.casefold() != expected_generator_model.casefold():
        raise ValueError(f"trace generator model {model!r} does not match {expected_generator_model!r}")
    mode = str(row.get("mode", "nonthinking")).strip()
    if mode not in ("thinking", "nonthinking"):
        raise ValueError(f"unsupported trace mode {mode!r}")
    if str(row.get("finish_reason", "stop")).strip() != "stop":
        raise ValueError(f"trace finish reason is not stop: {row.get('finish_reason')!r}")
    messages = row.get("messages")
    if not isinstance(messages, (list, tuple)) or not messages:
        raise TypeError("trace messages must be a non-empty sequence")
    out = []
    for m in messages:
        if not isinstance(m, Mapping) or str(m.get("role", "")) not in ("system", "user", "assistant", "tool") or "content" not in m:
            raise ValueError("every trace message needs a known role and content")
        out.append(dict(m))
    if out[-1]["role"] not in ("user", "tool"):
        raise ValueError("trace messages must end at a user query or tool response")
    output = row.get("output")
    if not isinstance(output, str) or not output.strip():
        raise ValueError("trace output must be a non-empty string")
    reasoning = row.get("reasoning") or ""
    if not isinstance(reasoning, str):
        raise TypeError("trace reasoning must be a string or null")
    if mode == "thinking" and not reasoning.strip():
        raise ValueError("thinking trace has no reasoning content")
    if mode == "nonthinking" and reasoning.strip():
        raise ValueError("nonthinking trace unexpectedly contains reasoning content")
    out.append({"role": "assistant", "content": output, "reasoning_content": reasoning})
    return out, mode, str(row.get("source_dataset", "unknown")).strip() or "unknown"


def build_trace_corpus(tokenizer: Any, output, rows: Iterable[Mapping[str, Any]], *, train_tokens: int, validation_tokens: int,
                       sequence_length: int = 4096, seed: int = 0, expected_generator_model: str | None = None,
                       source_files: Sequence[Path] = ()) -> CalibrationCorpus:
    """One window per trace: the prompt rendered with the generation prompt, then the generated turn; only generated
    positions are scored.  Traces longer than ``sequence_length`` or malformed are counted and left out; records are
    assigned to validation until its quota is met, then to train (after a seeded shuffle)."""
    rows = list(rows)
    order = np.random.default_rng(seed).permutation(len(rows))
    need = {"validation": int(validation_tokens), "train": int(train_tokens)}
    got = {"validation": 0, "train": 0}
    chunks, masks, split_ids, domain_ids = [], [], [], []
    domains: list[str] = []
    excluded: dict[str, int] = {}
    hashes = {s: [] for s in SPLITS}
    for i in order:
        split = "validation" if got["validation"] < need["validation"] else "train"
        if got[split] >= need[split]:
            break
        try:
            messages, mode, source = trace_record(rows[int(i)], expected_generator_model=expected_generator_model)
        except (TypeError, ValueError) as exc:
            excluded[type(exc).__name__ + ": " + str(exc)[:60]] = excluded.get(type(exc).__name__ + ": " + str(exc)[:60], 0) + 1
            continue
        prompt = tokenizer.apply_chat_template(messages[:-1], add_generation_prompt=True)
        full = tokenizer.apply_chat_template(messages, add_generation_prompt=False)
        if not full.startswith(prompt):  # a template that rewrites earlier turns: score the whole final turn conservatively
            prompt = full[: len(os.path.commonprefix([prompt, full]))]
        p_ids, f_ids = _encode(tokenizer, prompt), _encode(tokenizer, full)
        if len(f_ids) > sequence_length or len(f_ids) - len(p_ids) < 1 or len(f_ids) < 2:
            excluded["length"] = excluded.get("length", 0) + 1
            continue
        mask = np.zeros(len(f_ids), dtype=np.uint8)
        mask[max(1, len(p_ids)) :] = 1
        label = f"{source}/{mode}"
        if label not in domains:
            domains.append(label)
        chunks.append(np.asarray(f_ids, dtype=np.int32))
        masks.append(mask)
        split_ids.append(SPLITS[split])
        domain_ids.append(domains.index(label))
        got[split] += len(f_ids)
        hashes[split].append(hashlib.sha256(full.encode("utf-8")).hexdigest())
    if got["validation"] < min(need["validation"], 2) or got["train"] < min(need["train"], 2):
        raise ValueError(f"too few usable traces: {got} of {need} tokens (left out: {excluded})")
    manifest = {"format": MASKED_FORMAT, "seed": int(seed), "sequence_length": int(sequence_length), "domains": domains,
                "target_tokens": need, "actual_tokens": got, "scored_tokens": int(sum(int(m.sum()) for m in masks)),
                "record_sets": {s: {"count": len(hashes[s]), "sha256": hashlib.sha256("\n".join(hashes[s]).encode("ascii")).hexdigest()}
                                for s in SPLITS},
                "excluded": excluded, "tokenizer": _tokenizer_identity(tokenizer),
                "sources": {"files": [_file_identity(Path(p)) for p in source_files],
                            "expected_generator_model": expected_generator_model}}
    return _write(Path(output), chunks, split_ids, domain_ids, manifest, masks)
