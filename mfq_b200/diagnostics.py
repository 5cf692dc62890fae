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


def _prefill_logits(model, prompt: torch.Tensor) -> torch.Tensor:
    from .engine.llm_engine import LLMEngine
    from .models.llama import StepBuffers
    eng = LLMEngine(model, max_batch=1, max_seq_len=96, device="cpu")
    n = prompt.numel()
    eng.cache.assign(0, 7, n)
    step = StepBuffers(input_ids=prompt.to(torch.int32), positions=torch.arange(n, dtype=torch.int32),
                       slots=eng.cache.slots(7, 0, n), cu_seqlens=[0, n])
    return model.forward(step, eng.cache, prefill=True).float()


def _parallel_agreement(build, world: int, prompt: torch.Tensor) -> dict:
    """Logits of ``world`` in-process ranks (threads, CPU tensors) against the single-rank model."""
    from .parallel.local_collective import LocalGroup
    single = _prefill_logits(build(0, 1, None), prompt)
    ranks = LocalGroup(world).run(lambda rank, coll: _prefill_logits(build(rank, world, coll), prompt))
    same = all(torch.equal(r, ranks[0]) for r in ranks[1:])
    cos = float(torch.nn.functional.cosine_similarity(ranks[0].flatten(), single.flatten(), dim=0))
    return {"world": world, "ranks_identical": same, "cosine_vs_single": round(cos, 4), "ok": same and cos > 0.97}


def check_tp_linear() -> dict:
    """Tensor-parallel dense model (attention heads, FFN columns, vocabulary sharded over 2 and 4 ranks; 4 ranks on 2 KV
    heads replicate each head twice) against one rank.  Host-validated: ranks are threads over CPU tensors."""
    from .models.llama import LlamaConfig, LlamaModel, LlamaWeights
    cfg = LlamaConfig.tiny()
    prompt = torch.randint(0, cfg.vocab_size, (33,), generator=torch.Generator().manual_seed(33))
    build = lambda rank, w, coll: LlamaModel(cfg, LlamaWeights.random_init(cfg, "cpu", seed=3, std=0.05, tp_rank=rank, tp_size=w), collective=coll)
    res = [_parallel_agreement(build, w, prompt) for w in (2, 4)]
    return {"cases": res, "ok": all(r["ok"] for r in res)}


def check_ep_moe() -> dict:
    """Expert-parallel MoE decoder (experts split over 2 ranks, each adds its experts' partial) against one rank."""
    from .models.moe_decoder import MoeDecoderConfig, MoeDecoderModel, MoeWeights
    from .models.moe_lm import MoeConfig, init_weights
    cfg = MoeDecoderConfig.tiny()
    tensors = {k: v.numpy() for k, v in init_weights(MoeConfig(
        vocab_size=cfg.vocab_size, hidden_size=cfg.hidden_size, num_layers=cfg.num_layers, num_heads=cfg.num_heads,
        num_kv_heads=cfg.num_kv_heads, head_dim=cfg.head_dim, num_experts=cfg.num_experts, top_k=cfg.top_k,
        moe_intermediate=cfg.moe_intermediate, shared_intermediate=cfg.shared_intermediate), seed=4, std=0.05).items()}
    prompt = torch.randint(0, cfg.vocab_size, (29,), generator=torch.Generator().manual_seed(2))
    build = lambda rank, w, coll: MoeDecoderModel(cfg, MoeWeights.from_tensors(cfg, tensors, "cpu", rank, w), collective=coll)
    return _parallel_agreement(build, 2, prompt)


def check_continuous_batching(device: str | None = None) -> dict:
    """Requests that join and leave a running batch must generate what they generate alone (greedy)."""
    from .engine.llm_engine import LLMEngine
    from .engine.scheduler import ContinuousBatchScheduler, Request, SamplingParams
    from .models.llama import LlamaConfig, LlamaModel, LlamaWeights
    device = device or ("cuda" if torch.cuda.is_available() else "cpu")
    cfg = LlamaConfig.tiny()
    model = LlamaModel(cfg, LlamaWeights.random_init(cfg, device, seed=5, std=0.05))
    prompts = [list(range(3 + i, 20 + 4 * i)) for i in range(5)]

    def run(batch):
        eng = LLMEngine(model, max_batch=4, max_seq_len=128, device=device)
        sched = ContinuousBatchScheduler(eng, max_queue=16)
        reqs = [Request(list(p), SamplingParams(max_tokens=5 + 2 * i)) for i, p in enumerate(batch)]
        for r in reqs:
            sched.submit(r)
        for _ in range(400):
            if not sched.step() and sched.idle:
                break
        return [r.generated for r in reqs]

    together = run(prompts)  # five requests through four rows: the fifth joins when a row frees up
    alone = [run([p])[0][: len(t)] for p, t in zip(prompts, together)]
    same = sum(a == b[: len(a)] for a, b in zip(alone, together))
    # on a GPU a batch bucket changes the GEMM tile shape, so a near-tie may flip late in a sequence: first tokens must agree
    first = all(a[:1] == b[:1] for a, b in zip(alone, together))
    return {"requests": len(prompts), "identical": same, "first_tokens_agree": first,
            "ok": first and (same == len(prompts) or device != "cpu")}


def check_json_constraint() -> dict:
    """Grammar automaton + vocabulary mask (native library) on a byte vocabulary."""
    import json as _json
    from . import native
    vocab = native.JsonVocabulary([bytes([b]) for b in range(256)] + [b'{"', b'":', b"true", b"}}"])
    s = native.JsonState(vocab, need_object=True)
    doc = b'{"k": [1, 2.5e-1, {"z": null}], "s": "a\\n"}'
    ok = s.feed(doc) and s.complete and isinstance(_json.loads(doc), dict)
    t = native.JsonState(vocab, need_object=True)
    refused = not t.feed(b"[1]") and not t.feed(b'{"a" 1}')
    t.feed(b'{"a"')
    mask = t.mask()
    only_colon = bool(mask[ord(":")]) and not mask[ord("}")] and not mask[256]
    return {"accepts_valid": bool(ok), "refuses_invalid": refused, "mask": only_colon, "ok": bool(ok and refused and only_colon)}


CPU_CHECKS = {"nint": check_nint_roundtrip, "fp8-block": check_fp8_block_roundtrip, "tp-linear": check_tp_linear,
              "ep-moe": check_ep_moe, "continuous-batching": check_continuous_batching, "json-constraint": check_json_constraint}
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
