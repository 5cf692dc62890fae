"""Runs the benchmark's metric on the unmodified reference, through the reference's own runtime.

What runs: the reference's native CUDA runtime ``mfq-runtime`` (built from its unmodified ``cpp_runtime`` sources
for sm_100 with CMake by ``baseline/build_reference_runtime.sh``, binary kept in ``baseline/_ref/bin``), driven over its stdio NDJSON protocol exactly like its
own ``bench/model_bench.py`` does (``op: generate`` with ``benchmark_prompt_tokens``, cache disabled, greedy).  The
checkpoint is the same architecture and format as ours -- 32-layer 8B dense decoder, E4M3 weights with 128x128 fp32
block multipliers stored as all-SQ8 ``FP8-128SQ`` records -- written to a temporary ``.mfq`` with random-init
weights, loaded by the reference's stock ``qwen3_5`` text backbone (its dense Llama-style path).  The tokenizer
GGUF comes from the reference's own ``ensure_hf_tokenizer_gguf``.  None of this repository's kernels, models or
engine is on that path; this file only prepares data and speaks the protocol.

Differences that remain (the reference cannot express them): its KV cache is fp16 (it has no FP8 pages) and its
continuous batching is validated for at most 32 rows, so batch 64 is requested and whatever it accepts is reported.
"""

from __future__ import annotations

import json
import os
import queue
import subprocess
import sys
import tempfile
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
REF = ROOT / "_ref"
BINARY = REF / "bin" / "mfq-runtime"


def _unavailable(why: str) -> dict:
    return {"impl": "reference", "unavailable": why}


def _write_tokenizer(tmp: Path, vocab: int) -> Path:
    sys.path.insert(0, str(REF))
    from mfq.server.runtime.hf_tokenizer import ensure_hf_tokenizer_gguf
    src = tmp / "tok-src"
    src.mkdir()
    (src / "config.json").write_text(json.dumps({"model_type": "qwen3_5", "text_config": {"vocab_size": vocab}}))
    (src / "generation_config.json").write_text(json.dumps({"bos_token_id": vocab - 2, "eos_token_id": vocab - 1, "pad_token_id": vocab - 2}))
    (src / "tokenizer_config.json").write_text(json.dumps({"bos_token": "<bos>", "eos_token": "<eos>", "pad_token": "<bos>",
                                                            "chat_template": "{{ messages[0].content }}", "add_bos_token": False}))
    words = {"a": 0, "b": 1, "ab": 2}  # the GGUF converter wants at least one BPE merge
    words.update({f"t{i}": i for i in range(3, vocab - 2)})
    added = [{"id": vocab - 2 + j, "content": c, "special": True, "single_word": False, "lstrip": False, "rstrip": False,
              "normalized": False} for j, c in enumerate(("<bos>", "<eos>"))]
    (src / "tokenizer.json").write_text(json.dumps({"model": {"type": "BPE", "vocab": words, "merges": [["a", "b"]]}, "added_tokens": added}))
    return ensure_hf_tokenizer_gguf(src, tmp / "tok-cache")


def _write_model(path: Path, cfg: dict, device: str) -> None:
    """Random-init block-FP8 checkpoint in the reference's container, streamed tensor by tensor."""
    import numpy as np
    import torch
    sys.path.insert(0, str(ROOT.parent))
    from mfq_b200 import formats as F
    from mfq_b200.formats.container import ASSET_PREFIX, pack_tensor, write_streaming
    from mfq_b200.formats.fp8sq import block_fp8_tensor
    from mfq_b200.quantize.fp8_block import quantize_fp8_block_torch

    h, i, v = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    hq, hk, d, layers = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"], cfg["num_hidden_layers"]
    gen = torch.Generator(device=device).manual_seed(0)
    plan: list[tuple[str, tuple[int, ...], str]] = [("model.token_embedding.weight", (v, h), "bf16")]
    for l in range(layers):
        p = f"model.block.{l}."
        for name, shape in (("attention.query", (hq * d, h)), ("attention.key", (hk * d, h)), ("attention.value", (hk * d, h)),
                            ("attention.output", (h, hq * d)), ("mlp.gate", (i, h)), ("mlp.up", (i, h)), ("mlp.down", (h, i))):
            plan.append((p + name + ".weight", shape, "fp8"))
        for name, size in (("attention.norm", h), ("mlp.norm", h), ("attention.query_norm", d), ("attention.key_norm", d)):
            plan.append((p + name + ".weight", (size,), "zeros"))
    plan += [("model.output_norm.weight", (h,), "zeros"), ("model.output.weight", (v, h), "fp8")]

    def blob(shape, kind) -> tuple[str, bytes]:
        if kind == "zeros":  # the reference's Qwen RMSNorm stores (weight - 1)
            return pack_tensor(np.zeros(shape, np.float32))
        w = torch.randn(shape, generator=gen, device=device, dtype=torch.float32).mul_(0.02)
        if kind == "bf16":
            return pack_tensor(F.to_bf16(w.cpu().numpy()))
        q, s = quantize_fp8_block_torch(w)
        return pack_tensor(block_fp8_tensor(q.view(torch.uint8).cpu().numpy(), s.cpu().numpy()))

    graph = dict(schema_version=1, architecture="qwen3_5",
                 canonical_naming=dict(namespace="mfq.tensor", version=1, component_roots=["model"]),
                 topology=dict(text_layers=layers), graph=dict(kind="causal_lm", backbone="qwen3_5"),
                 components=[dict(kind="text", tensor_root="model", implementation="qwen3_5", policy="decoder")],
                 capabilities=["text"])
    assets = {ASSET_PREFIX + "model_config.json": json.dumps(cfg).encode(), ASSET_PREFIX + "model_graph.json": json.dumps(graph).encode()}
    # sizes first (one throw-away blob per distinct shape/kind), then stream the real blobs
    size_of: dict = {}
    for _n, shape, kind in plan:
        if (shape, kind) not in size_of:
            dt, b = blob(shape, kind)
            size_of[(shape, kind)] = (dt, len(b))
    items = [(n, *size_of[(shape, kind)]) for n, shape, kind in plan] + [(k, "BLOB", len(v_)) for k, v_ in assets.items()]

    def blobs():
        for _n, shape, kind in plan:
            yield blob(shape, kind)[1]
        for v_ in assets.values():
            yield v_
    write_streaming(path, F.FileHeader(version=2, model_arch="qwen3_5"), items, blobs())


class _Runtime:
    def __init__(self, cmd, env) -> None:
        self.proc = subprocess.Popen(cmd, stdin=subprocess.PIPE, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True,
                                     bufsize=1, env=env, start_new_session=True)
        self.lines: "queue.Queue[str | None]" = queue.Queue()
        self.tail: list[str] = []
        threading.Thread(target=self._out, daemon=True).start()
        threading.Thread(target=self._err, daemon=True).start()

    def _out(self):
        for line in self.proc.stdout:
            self.lines.put(line)
        self.lines.put(None)

    def _err(self):
        for line in self.proc.stderr:
            self.tail.append(line.rstrip()[:300])
            del self.tail[:-30]

    def read(self, timeout: float) -> dict:
        deadline = time.monotonic() + timeout
        while True:
            line = self.lines.get(timeout=max(0.01, deadline - time.monotonic()))
            if line is None:
                raise RuntimeError("reference runtime closed its output: " + " | ".join(self.tail[-5:]))
            if line.strip():
                return json.loads(line)

    def send(self, frame: dict) -> None:
        self.proc.stdin.write(json.dumps(frame) + "\n")
        self.proc.stdin.flush()

    def close(self) -> None:
        try:
            self.proc.stdin.close()
            self.proc.wait(timeout=20)
        except Exception:
            self.proc.kill()  # the exact process this object started


def _generate(rt: _Runtime, ids: list[str], prompt_tokens: int, new_tokens: int, timeout: float) -> dict[str, dict]:
    for rid in ids:
        rt.send({"v": 1, "id": rid, "op": "generate", "params": {
            "model": "bench", "input": {"messages": [{"role": "user", "content": "ab"}], "preformatted_prompt": "ab",
                                        "benchmark_prompt_tokens": prompt_tokens},
            "cache": {"enabled": False}, "sampling": {"temperature": 0.0, "max_new_tokens": new_tokens, "seed": 1, "enable_mtp": False},
            "stream": False}})
    results: dict[str, dict] = {}
    done: set[str] = set()
    deadline = time.monotonic() + timeout
    while len(done) < len(ids):
        msg = rt.read(deadline - time.monotonic())
        rid = msg.get("id")
        if rid not in ids:
            continue
        if msg.get("type") == "error":
            raise RuntimeError(str(msg)[:300])
        data = msg.get("data", msg)
        if isinstance(data, dict) and "metrics" in data:
            results[rid] = data
        if msg.get("type") == "done":
            done.add(rid)
    return results


def run(args) -> dict:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return {}  # the reference drives all GPUs from one process
    if not BINARY.exists():
        return _unavailable("reference native runtime binary is not present under baseline/_ref/bin (CMake build of cpp_runtime for sm_100)")
    try:
        import torch
        if not torch.cuda.is_available():
            return _unavailable("no CUDA device")
        tiny = getattr(args, "tiny", False)
        cfg = dict(model_type="qwen3_5", hidden_size=256 if tiny else 4096, vocab_size=1024 if tiny else 128256,
                   intermediate_size=512 if tiny else 14336, num_hidden_layers=2 if tiny else 32,
                   num_attention_heads=4 if tiny else 32, num_key_value_heads=2 if tiny else 8, head_dim=128,
                   max_position_embeddings=8192, layer_types=["full_attention"] * (2 if tiny else 32),
                   rope_theta=5e5, rms_norm_eps=1e-5, eos_token_id=(1024 if tiny else 128256) - 1, tie_word_embeddings=False)
        # the reference refuses more than 32 concurrent sequences ("continuous batching sequence limit must be in
        # [1, 32]; 64 is not validated"), so its arm runs at the largest batch it accepts
        # 256 generated tokens per request, as the benchmark configuration names (the driver's --steps / --warmup describe
        # our arm's graph replays; here a longer run also keeps the batch ramp-up a small part of the measurement)
        batch, ctx, new = min(args.batch, 32), args.context, 16 if tiny else 256
        with tempfile.TemporaryDirectory(prefix="mfq-ref-") as td:
            tmp = Path(td)
            tok = _write_tokenizer(tmp, cfg["vocab_size"])
            model = tmp / "llama8b-fp8.mfq"
            _write_model(model, cfg, "cuda")
            cmd = [str(BINARY), "--model", str(model), "--tokenizer", str(tok), "--transport", "stdio", "--ctx-size", str(ctx + new + 64),
                   "--continuous-batching", str(batch)]
            if args.gpus > 1:
                cmd += ["--tensor-parallel", ",".join(str(i) for i in range(args.gpus))]
            env = dict(os.environ, MFQ_RUNTIME_DISABLE_PREFIX_CACHE="1")
            rt = _Runtime(cmd, env)
            try:
                greet = rt.read(900)
                if greet.get("type") != "ready":
                    return _unavailable(f"reference runtime did not start: {str(greet)[:200]}")
                _generate(rt, ["warm"], min(ctx, 256), 4, 900)
                single = _generate(rt, ["one"], ctx, new, 3600)["one"]
                t0 = time.monotonic()
                many = _generate(rt, [f"r{i}" for i in range(batch)], ctx, new, 7200)
                wall = time.monotonic() - t0
            finally:
                rt.close()
        dec_tokens = sum(r["usage"]["completion_tokens"] - 1 for r in many.values())
        all_tokens = sum(r["usage"]["completion_tokens"] for r in many.values())
        # The runtime prefills the requests one after another and interleaves decode steps; a request's own decode_ms
        # therefore contains the other requests' prefills.  Aggregate decode rate = decode tokens over the wall time
        # that was not spent in (serialized) prefill.
        prefill_s = sum(r["metrics"]["prefill_ms"] for r in many.values()) / 1e3
        dec_s = max(wall - prefill_s, 1e-3)
        dec_ms = dec_s * 1e3
        value = dec_tokens / dec_s
        m1 = single["metrics"]
        return {
            "impl": "reference", "metric": "decode_tok_s_bs64", "value": round(value, 2), "unit": "tok/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(dec_ms / max(1, new - 1), 4), "higher_is_better": True,
            "scaling": "strong", "vs_baseline": round(value / 156.56, 2), "dtype": "fp8_e4m3 weights (decoded to fp16 in its kernels), fp16 KV",
            "data": "synthetic (benchmark_prompt_tokens, random-init N(0,0.02) weights)",
            "config": {"model": "llama-8b-fp8 (reference qwen3_5 backbone)", "global_batch": batch, "seq_len": ctx,
                       "parallelism": f"tp{args.gpus}", "requests_completed": len(many), "wall_s": round(wall, 2),
                       "batch_note": "requested %d; the reference accepts at most 32 concurrent sequences" % args.batch,
                       "decode_tokens_per_request": new,
                       "method": "decode tokens of all concurrent requests / (wall time - sum of their reported prefill_ms)"},
            # The figure above already IS end to end: it is wall-clock time around the reference's public protocol (requests in
            # over stdin, tokens out over stdout), with the serialized prefill time the runtime reports taken out so that it
            # is a decode rate like ours; token ids in and out are the host <-> device traffic of a step.
            "e2e": {"value": round(value, 2), "unit": "tok/s", "h2d_bytes_per_step": batch * 4, "d2h_bytes_per_step": batch * 4,
                    "with_prefill_tok_s": round(all_tokens / wall, 2)},
            "extra": {"decode_tok_s_bs1": round((single["usage"]["completion_tokens"] - 1) * 1e3 / m1["decode_ms"], 2),
                      "prefill_tok_s": round(ctx * 1e3 / m1["prefill_ms"], 1), "prefill_ms": round(m1["prefill_ms"], 2)},
        }
    except Exception as exc:  # a reference that cannot run this config is reported, not raised
        return _unavailable(f"reference run failed: {type(exc).__name__}: {str(exc)[:240]}")
