"""Model-level benchmark: drive a runtime over its stdio protocol with prompts of exact token counts.

For every (prompt length, concurrency) cell the driver sends ``concurrency`` ``generate`` frames at once -- each asks
for ``benchmark_prompt_tokens`` synthetic prompt tokens and a fixed number of new tokens, greedy -- waits for all the
results, repeats, and keeps the median of: time to first token, prefill tokens/s (per request), decode tokens/s per
request, and the aggregate generated tokens/s of the cell (all completions over the wall time of the cell).  The
result is one JSON document, renderable as Markdown or a self-contained HTML page.

The child is any command that speaks the version-1 frames (``mfq runtime --model x.mfq`` of this package, or the
reference's ``mfq-runtime --transport stdio``); environment variables pass through, so GPU selection and runtime knobs
are the caller's.  Reference: ``bench/model_bench.py`` (driver) and ``bench/render_model_report.py`` (report).
"""

from __future__ import annotations

import html
import json
import queue
import statistics
import subprocess
import threading
import time


class RuntimeClient:
    """A runtime child process and its frame streams."""

    def __init__(self, command: list[str], env: dict | None = None, ready_timeout: float = 600.0) -> None:
        self.proc = subprocess.Popen(command, stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True, bufsize=1, env=env)
        self._frames: "queue.Queue[dict | None]" = queue.Queue()
        self._reader = threading.Thread(target=self._read, daemon=True)
        self._reader.start()
        self._n = 0
        first = self._next(ready_timeout)
        if first.get("type") != "ready":
            raise RuntimeError(f"runtime did not announce itself: {first}")
        self.ready = first

    def _read(self) -> None:
        for line in self.proc.stdout:
            line = line.strip()
            if line.startswith("{"):
                try:
                    self._frames.put(json.loads(line))
                except ValueError:
                    pass
        self._frames.put(None)

    def _next(self, timeout: float) -> dict:
        try:
            frame = self._frames.get(timeout=timeout)
        except queue.Empty:
            raise TimeoutError(f"no frame from the runtime within {timeout:.0f} s") from None
        if frame is None:
            raise RuntimeError(f"runtime exited (code {self.proc.poll()})")
        return frame

    def send(self, frame: dict) -> None:
        self.proc.stdin.write(json.dumps({"v": 1, **frame}) + "\n")
        self.proc.stdin.flush()

    def generate_many(self, requests: list[dict], timeout: float = 600.0) -> list[dict]:
        """Send all ``params`` dictionaries at once; returns their ``result`` data in the same order."""
        ids = []
        for params in requests:
            self._n += 1
            ids.append(f"bench-{self._n}")
            self.send({"id": ids[-1], "op": "generate", "params": params})
        results, open_ids = {}, set(ids)
        deadline = time.monotonic() + timeout
        while open_ids:
            frame = self._next(max(0.1, deadline - time.monotonic()))
            rid = frame.get("id")
            if rid not in open_ids and rid not in results:
                continue
            if frame["type"] == "error":
                raise RuntimeError(f"request {rid} failed: {frame.get('error')}")
            if frame["type"] == "result":
                results[rid] = frame["data"]
            elif frame["type"] == "done":
                open_ids.discard(rid)
        return [results[i] for i in ids]

    def close(self) -> None:
        try:
            self.send({"op": "shutdown"})
            self.proc.stdin.close()
            self.proc.wait(timeout=60)
        except Exception:
            self.proc.kill()


def _params(prompt_tokens: int, new_tokens: int, model: str | None, mtp: bool) -> dict:
    p = {"input": {"benchmark_prompt_tokens": prompt_tokens}, "cache": {"enabled": False}, "stream": False,
         "sampling": {"temperature": 0.0, "max_new_tokens": new_tokens, "seed": 0, "enable_mtp": mtp}}
    if model:
        p["model"] = model
    return p


def run_matrix(client: RuntimeClient, prompt_lengths: list[int], new_tokens: int, concurrency: list[int], repeats: int = 3,
               warmup: int = 1, model: str | None = None, mtp: bool = False) -> list[dict]:
    rows = []
    for n in prompt_lengths:
        for c in concurrency:
            reqs = [_params(n, new_tokens, model, mtp) for _ in range(c)]
            for _ in range(warmup):
                client.generate_many(reqs)
            samples = []
            for _ in range(repeats):
                t0 = time.monotonic()
                res = client.generate_many(reqs)
                wall = time.monotonic() - t0
                m = [r["metrics"] for r in res]
                done = sum(r["usage"]["completion_tokens"] for r in res)
                samples.append({"ttft_ms": statistics.median(x["ttft_ms"] for x in m),
                                "prefill_tps": statistics.median(x["prefill_tps"] for x in m),
                                "decode_tps": statistics.median(x["decode_tps"] for x in m),
                                "aggregate_tps": done / wall, "completion_tokens": done, "wall_s": wall})
            row = {"prompt_tokens": n, "new_tokens": new_tokens, "concurrency": c, "repeats": repeats}
            for k in ("ttft_ms", "prefill_tps", "decode_tps", "aggregate_tps", "wall_s"):
                row[k] = statistics.median(s[k] for s in samples)
            row["completion_tokens"] = samples[-1]["completion_tokens"]
            rows.append(row)
    return rows


def benchmark(command: list[str], prompt_lengths, new_tokens, concurrency, repeats=3, warmup=1, model=None, mtp=False,
              env=None, label: str = "") -> dict:
    client = RuntimeClient(command, env=env)
    try:
        rows = run_matrix(client, list(prompt_lengths), new_tokens, list(concurrency), repeats, warmup, model, mtp)
    finally:
        client.close()
    return {"format": "mfq.model-bench.v1", "label": label, "command": command, "models": client.ready.get("data", {}).get("models"),
            "mtp": mtp, "rows": rows}


def validate_report(report: dict) -> list[str]:
    """Problems that make a benchmark report unusable (empty list: fine).  Checked before a report is rendered or
    compared: every cell present once, positive rates, completions within what was asked for."""
    problems = []
    if report.get("format") != "mfq.model-bench.v1":
        problems.append(f"unknown format {report.get('format')!r}")
    seen = set()
    for i, r in enumerate(report.get("rows") or []):
        cell = (r.get("prompt_tokens"), r.get("concurrency"), r.get("new_tokens"))
        if cell in seen:
            problems.append(f"row {i}: cell {cell} appears twice")
        seen.add(cell)
        for key in ("ttft_ms", "prefill_tps", "aggregate_tps"):
            v = r.get(key)
            if not isinstance(v, (int, float)) or not v > 0 or v != v or v == float("inf"):
                problems.append(f"row {i}: {key} = {v!r}")
        done, asked = r.get("completion_tokens", 0), (r.get("new_tokens") or 0) * (r.get("concurrency") or 0)
        if not 0 < done <= asked:
            problems.append(f"row {i}: {done} completion tokens for {asked} asked")
    if not report.get("rows"):
        problems.append("no rows")
    return problems


# ---- reports ---------------------------------------------------------------------------------------------------------
_COLUMNS = (("prompt_tokens", "prompt", "{:d}"), ("concurrency", "streams", "{:d}"), ("new_tokens", "new", "{:d}"),
            ("ttft_ms", "TTFT ms", "{:.1f}"), ("prefill_tps", "prefill tok/s", "{:.0f}"),
            ("decode_tps", "decode tok/s per stream", "{:.1f}"), ("aggregate_tps", "generated tok/s, all streams", "{:.1f}"))


def render_markdown(report: dict) -> str:
    lines = [f"# Model benchmark {report.get('label') or ''}".rstrip(), "",
             "| " + " | ".join(c[1] for c in _COLUMNS) + " |", "|" + "---|" * len(_COLUMNS)]
    for r in report["rows"]:
        lines.append("| " + " | ".join(fmt.format(r[key]) for key, _h, fmt in _COLUMNS) + " |")
    lines += ["", f"command: `{' '.join(report['command'])}`", ""]
    return "\n".join(lines)


def render_html(report: dict) -> str:
    """One self-contained page: the table plus a bar per cell scaled to the best aggregate rate."""
    best = max((r["aggregate_tps"] for r in report["rows"]), default=1.0) or 1.0
    head = "".join(f"<th>{html.escape(h)}</th>" for _k, h, _f in _COLUMNS)
    body = []
    for r in report["rows"]:
        cells = "".join(f"<td>{html.escape(fmt.format(r[key]))}</td>" for key, _h, fmt in _COLUMNS)
        body.append(f"<tr>{cells}<td class=bar><div style='width:{100 * r['aggregate_tps'] / best:.1f}%'></div></td></tr>")
    style = ("body{font:14px system-ui;margin:2em}table{border-collapse:collapse}td,th{padding:4px 10px;border-bottom:1px solid #ddd;"
             "text-align:right}td.bar{width:220px}td.bar div{height:10px;background:#4a7}")
    return (f"<!doctype html><html><head><meta charset=utf-8><title>Model benchmark</title><style>{style}</style></head><body>"
            f"<h1>Model benchmark {html.escape(report.get('label') or '')}</h1><table><tr>{head}<th></th></tr>{''.join(body)}</table>"
            f"<p><code>{html.escape(' '.join(report['command']))}</code></p></body></html>")
