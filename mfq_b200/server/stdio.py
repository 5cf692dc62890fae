"""stdio transport: newline-delimited JSON frames on stdin / stdout (version 1 of the reference's private protocol).

A driver that speaks to the reference's ``mfq-runtime --transport stdio`` (its bench harness does,
``bench/model_bench.py``; framing in ``cpp_runtime/transport/stdio.cpp``) can speak to this runtime the same way:

    <- {"v": 1, "type": "ready", "data": {"models": [...]}}                        once, at start
    -> {"v": 1, "id": "r1", "op": "generate", "params": {"model": .., "input": {"messages": [...] | "preformatted_prompt":
        "...", "benchmark_prompt_tokens": N}, "sampling": {"temperature", "top_p", "top_k", "max_new_tokens", "seed",
        "enable_mtp"}, "stream": bool}}
    <- {"v": 1, "id": "r1", "type": "delta", "data": {"text": "..."}}              (stream only)
    <- {"v": 1, "id": "r1", "type": "result", "data": {"text", "finish_reason", "usage", "metrics"}}
    <- {"v": 1, "id": "r1", "type": "done"}
    -> {"op": "cancel", "params": {"target": "r1"}}, {"op": "status"}, {"op": "shutdown"}

``input.token_ids`` gives an exact, already tokenized prompt; ``"stream_tokens": true`` adds one
``{"type": "token", "data": {"id": N}}`` frame per generated token (stop tokens included), which is what a front-end
process that owns the tokenizer and proxies requests to worker processes consumes (``server/worker.py``).

``benchmark_prompt_tokens`` replaces the prompt by exactly that many synthetic token ids (what benchmarks use to pin the
prompt length).  Requests run concurrently: every ``generate`` gets a thread that forwards its events; one lock
serialises the writes, so frames never interleave inside a line.
"""

from __future__ import annotations

import json
import queue
import threading
import time

from ..engine.scheduler import SamplingParams


class StdioTransport:
    def __init__(self, service, reader, writer) -> None:
        self.service, self.reader, self.writer = service, reader, writer
        self._lock = threading.Lock()
        self._threads: list[threading.Thread] = []
        self._requests: dict[str, tuple[object, object]] = {}  # id -> (model, request)

    def send(self, frame: dict) -> None:
        with self._lock:
            self.writer.write(json.dumps({"v": 1, **frame}) + "\n")
            self.writer.flush()

    # ---- operations ------------------------------------------------------------------------------------------------
    def _prompt_ids(self, lm, params: dict) -> list[int]:
        inp = params.get("input") or {}
        if inp.get("token_ids"):  # an exact prompt, already tokenized (a front end that owns the tokenizer)
            return [int(t) for t in inp["token_ids"]]
        n = int(inp.get("benchmark_prompt_tokens") or 0)
        if n > 0:
            vocab = getattr(lm.tokenizer, "vocab_size", 256)
            return [3 + (i * 7919) % max(1, vocab - 8) for i in range(n)]
        if inp.get("preformatted_prompt"):
            return lm.tokenizer.encode(inp["preformatted_prompt"])
        return lm.tokenizer.encode(lm.tokenizer.apply_chat_template(inp.get("messages") or [], add_generation_prompt=True))

    def _generate(self, rid: str, params: dict) -> None:
        try:
            lm = self.service.resolve(params.get("model"))
            s = params.get("sampling") or {}
            stops = tuple(int(t) for t in s["stop_token_ids"]) if "stop_token_ids" in s else tuple(lm.tokenizer.stop_ids)
            sp = SamplingParams(max_tokens=int(s.get("max_new_tokens", 256)), temperature=float(s.get("temperature", 0.0)),
                                top_p=float(s.get("top_p", 1.0)), top_k=int(s.get("top_k", 0)), seed=int(s.get("seed", 0)),
                                presence_penalty=float(s.get("presence_penalty", 0.0)), frequency_penalty=float(s.get("frequency_penalty", 0.0)),
                                repetition_penalty=float(s.get("repetition_penalty", 1.0)),
                                stop_token_ids=stops, enable_mtp=bool(s.get("enable_mtp", False)),
                                response_format=params.get("response_format") or None,
                                logit_bias={int(k): float(v) for k, v in (params.get("logit_bias") or {}).items()} or None)
            ids = self._prompt_ids(lm, params)
            t0 = time.monotonic()
            req, events = self.service.submit(lm, ids, sp, priority=int(params.get("priority", 0) or 0),
                                              timeout_seconds=params.get("timeout_seconds"))
        except KeyError as exc:
            return self._fail(rid, "model_not_found", f"model {exc.args[0]!r} is not loaded")
        except Exception as exc:  # queue full, invalid parameters, ...
            return self._fail(rid, getattr(exc, "code", "invalid_request"), str(exc))
        self._requests[rid] = (lm, req)
        out, text, first, finish, error = [], "", None, None, None
        while True:
            try:
                ev = events.get(True, 0.25)
            except queue.Empty:
                continue
            if ev.kind == "token":
                first = first or time.monotonic()
                if params.get("stream_tokens"):  # raw ids, stop tokens included: the front end decodes
                    self.send({"id": rid, "type": "token", "data": {"id": int(ev.token)}})
                if ev.token in sp.stop_token_ids:
                    continue
                out.append(ev.token)
                full = lm.tokenizer.decode(out)
                piece, text = full[len(text):], full
                if params.get("stream") and piece:
                    self.send({"id": rid, "type": "delta", "data": {"text": piece}})
            elif ev.kind == "completed":
                finish = ev.finish_reason
                break
            elif ev.kind == "failed":
                error = ev.error_code
                break
        self._requests.pop(rid, None)
        if error:
            return self._fail(rid, error, "generation failed")
        end = time.monotonic()
        first = first or end
        self.send({"id": rid, "type": "result", "data": {
            "text": text, "finish_reason": finish or "stop",
            "usage": {"prompt_tokens": len(ids), "completion_tokens": len(out), "total_tokens": len(ids) + len(out)},
            "metrics": self._metrics(len(ids), len(out), t0, first, end)}})
        self.send({"id": rid, "type": "done"})

    @staticmethod
    def _metrics(prompt: int, completion: int, t0: float, first: float, end: float) -> dict:
        """Per-request timing as the reference runtime reports it (``InferenceMetrics``: ttft, prefill / decode ms and
        rates).  The first generated token belongs to the prefill; decode covers the tokens after it."""
        prefill_ms, decode_ms = (first - t0) * 1e3, (end - first) * 1e3
        return {"prompt_tokens": prompt, "prefill_tokens": prompt, "completion_tokens": completion,
                "ttft_ms": prefill_ms, "prefill_ms": prefill_ms, "decode_ms": decode_ms, "total_ms": (end - t0) * 1e3,
                "prefill_tps": prompt / max(prefill_ms, 1e-6) * 1e3,
                "decode_tps": max(completion - 1, 0) / max(decode_ms, 1e-6) * 1e3,
                "generation_tps": completion / max((end - t0) * 1e3, 1e-6) * 1e3}

    def _fail(self, rid, code: str, message: str) -> None:
        self.send({"id": rid, "type": "error", "error": {"code": code, "message": message}})
        self.send({"id": rid, "type": "done"})

    # ---- loop --------------------------------------------------------------------------------------------------------
    def serve(self) -> None:
        self.send({"type": "ready", "data": {"models": list(self.service.models), "protocol": "ndjson.v1"}})
        for line in self.reader:
            line = line.strip()
            if not line:
                continue
            try:
                frame = json.loads(line)
            except ValueError:
                self.send({"type": "error", "error": {"code": "invalid_frame", "message": "not a JSON line"}})
                continue
            op, rid, params = frame.get("op"), frame.get("id"), frame.get("params") or {}
            if op == "generate":
                t = threading.Thread(target=self._generate, args=(str(rid), params), daemon=True)
                t.start()
                self._threads.append(t)
            elif op == "cancel":
                target = self._requests.get(str(params.get("target")))
                if target:
                    self.service.cancel(target[0], target[1].id)
                self.send({"id": rid, "type": "result", "data": {"cancelled": bool(target)}})
            elif op == "status":
                self.send({"id": rid, "type": "result", "data": self.service.status()})
            elif op == "shutdown":
                break
            else:
                self.send({"id": rid, "type": "error", "error": {"code": "unknown_op", "message": f"unknown op {op!r}"}})
        for t in self._threads:
            t.join(timeout=60)
