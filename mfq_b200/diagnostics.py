"""``mfq diagnose``: self-checks a user can run on a box before serving.

Every check compares one component against its plain fp32 restatement (the same oracles the test-suite uses) and
reports the largest error relative to the magnitude of the expected values.  Format checks run anywhere; kernel checks
need a B200 and the built extension.  Nothing here provokes a fault: inputs are valid and every kernel wait is bounded.
Reference: ``cpp_runtime/backends/cuda/diagnostics`` (the ``mfq-diagnostics --check-* / --compare-*`` executable).
"""

from __future__ import annotations

import json
import math
import time

import numpy as np
import torch


def _rel(got: torch.Tensor, want: torch.Tensor) -> float:
    return float((got.float() - want.float()).abs().max() / (want.float().abs().max() + 1e-6))


# ---- format checks (CPU) --------------------------------------------------------------------------------------------
def check_nint_roundtrip() -> dict:
    from . import formats as F
    from .quantize import nint
    rng = np.random.default_rng(0)
    w = rng.standard_normal((64, 256)).astype(np.float32)
    t = nint.quantize_nint(w, nint.NintSpec())
    back = np.asarray(F.dequantize(t), dtype=np.float32)
    snr = 10 * math.log10(float((w ** 2).sum() / ((w - back) ** 2).sum()))
    return {"snr_db": round(snr, 2), "ok": snr > 18.0}


def check_fp8_block_roundtrip() -> dict:
    from .quantize.fp8_block import dequantize_fp8_block_torch, quantize_fp8_block_torch
    w = torch.randn((256, 384), generator=torch.Generator().manual_seed(0)) * 0.02
    q, s = quantize_fp8_block_torch(w)
    err = _rel(dequantize_fp8_block_torch(q, s), w)
    return {"rel_err": round(err, 4), "ok": err < 0.07}


def check_container(tmp_dir) -> dict:
    from . import formats as F
    path = f"{tmp_dir}/diag.mfq"
    a = np.arange(24, dtype=np.float32).reshape(4, 6)
    F.save(path, F.FileHeader(model_arch="diag"), {"a": a, "__mfq_asset__/x.json": b"{}"})
    with F.open_mfq(path) as store:
        ok = np.array_equal(np.asarray(F.dequantize(store["a"])), a) and store.assets()["x.json"] == b"{}"
    return {"ok": bool(ok)}


# ---- kernel checks (GPU) --------------------------------------------------------------------------------------------
def _gemm_case(m, n, k, seed=0):
    from .ops import reference as ref
    from .quantize.fp8_block import quantize_fp8_block_torch
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn((m, k), generator=g, device="cuda").to(torch.bfloat16)
    w = (torch.randn((n, k), generator=g, device="cuda") * 0.05).to(torch.bfloat16)
    return (*ref.quant_rows(x), *quantize_fp8_block_torch(w))


def check_fp8_gemm() -> dict:
    from . import ops
    from .ops import reference as ref
    worst = 0.0
    for m, n, k in ((64, 512, 1024), (300, 640, 1536), (1, 4096, 4096), (16, 1040, 512)):
        xq, xs, wq, ws = _gemm_case(m, n, k)
        worst = max(worst, _rel(ops.fp8_gemm(xq, xs, wq, ws), ref.fp8_gemm(xq, xs, wq, ws)))
    return {"rel_err": round(worst, 4), "ok": worst < 2e-2}


def check_attention() -> dict:
    from .ops import kernels as K
    from .ops import reference as ref
    worst = 0.0
    for d, hq, hk in ((128, 8, 2), (256, 4, 1)):
        g = torch.Generator(device="cuda").manual_seed(d)
        q = torch.randn((300, hq, d), generator=g, device="cuda").to(torch.bfloat16)
        k = torch.randn((377, hk, d), generator=g, device="cuda").to(torch.bfloat16)
        v = torch.randn((377, hk, d), generator=g, device="cuda").to(torch.bfloat16)
        sc = 1 / math.sqrt(d)
        worst = max(worst, _rel(K.attn_prefill_bf16(q, k, v, sc), ref.attention(q, k, v, sc, causal_offset=77)))
    return {"rel_err": round(worst, 4), "ok": worst < 2e-2}


def check_engine_greedy() -> dict:
    """CUDA-graph decode and eager decode of a tiny model must produce the same tokens (same kernels, same order), and
    the first token must be the one the CPU reference path picks unless its two best logits are nearly tied."""
    from .engine.llm_engine import LLMEngine
    from .models.llama import LlamaConfig, LlamaModel, LlamaWeights
    cfg = LlamaConfig.tiny()
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=torch.Generator().manual_seed(n)) for n in (33, 17)]
    model = LlamaModel(cfg, LlamaWeights.random_init(cfg, "cuda", seed=5, std=0.05))
    graph = LLMEngine(model, max_batch=2, max_seq_len=128).generate(prompts, 6).tokens
    eager = LLMEngine(model, max_batch=2, max_seq_len=128, use_graphs=False).generate(prompts, 6).tokens
    return {"graph_equals_eager": bool(torch.equal(graph, eager)), "ok": bool(torch.equal(graph, eager))}


CPU_CHECKS = {"nint": check_nint_roundtrip, "fp8-block": check_fp8_block_roundtrip}
GPU_CHECKS = {"fp8-gemm": check_fp8_gemm, "attention": check_attention, "engine": check_engine_greedy}


def run(names: list[str] | None = None, tmp_dir: str | None = None) -> dict:
    import tempfile
    report = {"cuda": torch.cuda.is_available(), "checks": {}}
    todo = dict(CPU_CHECKS)
    todo["container"] = lambda: check_container(tmp_dir or tempfile.mkdtemp(prefix="mfq-diag-"))
    if torch.cuda.is_available():
        todo.update(GPU_CHECKS)
    for name, fn in todo.items():
        if names and name not in names:
            continue
        t0 = time.time()
        try:
            res = fn()
        except Exception as exc:  # a check that cannot run is a failed check, reported with its reason
            res = {"ok": False, "error": f"{type(exc).__name__}: {exc}"}
        res["seconds"] = round(time.time() - t0, 3)
        report["checks"][name] = res
    if torch.cuda.is_available():
        from .ops import Workspace
        torch.cuda.synchronize()
        try:
            Workspace.get(torch.device("cuda", torch.cuda.current_device())).check()
            report["device_status"] = "clean"
        except Exception as exc:
            report["device_status"] = str(exc)
    report["ok"] = all(c["ok"] for c in report["checks"].values()) and report.get("device_status", "clean") == "clean"
    return report


def main(args) -> int:
    report = run(args.check or None)
    print(json.dumps(report, indent=1))
    return 0 if report["ok"] else 1
