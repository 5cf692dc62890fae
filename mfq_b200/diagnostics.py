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



# ---- more self-checks: every codec, the native helpers, the newer kernels --------------------------------------------------
def _w(rows=32, cols=256, seed=0, scale=0.05):
    return (np.random.default_rng(seed).normal(size=(rows, cols)) * scale).astype(np.float32)


def _rel_np(got, want) -> float:
    return float(np.abs(np.asarray(got, dtype=np.float64) - want).max() / (np.abs(want).max() + 1e-12))


def check_codecs() -> dict:
    """Quantize -> pack -> unpack -> dequantize for every weight family: bytes are stable, errors are at their family's level."""
    from . import formats as F
    from .formats import npq0
    from .quantize.expertwise import parse_profiles, quantize_matrix
    w = _w()
    out, ok = {}, True
    limits = {"NINT2": 0.6, "NINT3": 0.3, "NINT4": 0.15, "NINT5": 0.08, "NINT6": 0.04, "NINT8": 0.02, "NVQ3": 0.5, "MXFP4": 0.2,
              "FP8": 0.07, "NPQ0-S": 1.5, "NPQ0-L": 1.5, "NVQ1-L": 1.2, "NVQ1-S": 1.2,
              "NEPQ0-S": 1.5, "NEPQ1-S": 1.2, "NEPQ1-A": 1.2}
    for fam, lim in limits.items():
        t = quantize_matrix(w, parse_profiles(fam)[0])
        dtype, blob = F.pack_tensor(t)
        again = F.pack_tensor(F.unpack_tensor(dtype, blob))[1]
        err = _rel_np(F.dequantize(F.unpack_tensor(dtype, blob)).reshape(w.shape), w)
        good = again == blob and err <= lim
        ok &= good
        out[fam] = {"bytes": len(blob), "bits_per_weight": round(8 * len(blob) / w.size, 3), "max_rel_err": round(err, 4), "ok": good}
    return {"ok": ok, "families": out}


def check_mfe_and_expert_mix() -> dict:
    from . import formats as F
    from .quantize.expertwise import balanced_expert_mix, parse_profiles, quantize_expertwise
    w = np.stack([_w(16, 128, seed=e) for e in range(6)])
    profiles = parse_profiles("NINT4,NVQ3,MXFP4")
    assign = balanced_expert_mix("model.block.0.mlp.experts.up.weight", 6, 3, 7)
    t = quantize_expertwise(w, assign, profiles)
    dtype, blob = F.pack_tensor(t)
    rec = F.dequantize(F.unpack_tensor(dtype, blob))
    counts = np.bincount(assign, minlength=3).tolist()
    return {"ok": dtype == "MFE" and rec.shape == w.shape and counts == [2, 2, 2] and _rel_np(rec, w) < 0.6,
            "per_family": counts, "max_rel_err": round(_rel_np(rec, w), 4)}


def check_fp8_sq_palettes() -> dict:
    from .formats.fp8sq import block_fp8_tensor, dequantize_fp8sq
    from .quantize.fp8_block import quantize_fp8_block
    from .quantize.fp8_sq import quantize_fp8_sq
    w = _w(128, 256)
    base = block_fp8_tensor(quantize_fp8_block(w)) if hasattr(quantize_fp8_block(w), "q") else quantize_fp8_block(w)
    full = dequantize_fp8sq(base)
    errs = {}
    for bits in (7.0, 5.0, 3.0):
        errs[bits] = _rel_np(dequantize_fp8sq(quantize_fp8_sq(base, bits)), full)
    mono = errs[7.0] <= errs[5.0] <= errs[3.0]
    return {"ok": mono and errs[7.0] < 0.1, "max_rel_err_by_bits": {str(k): round(v, 4) for k, v in errs.items()}}


def check_gguf_blocks() -> dict:
    """Block and super-block GGUF types decode to finite numbers of the right count (bit-equality with the `gguf` package is a
    unit test; this runs anywhere)."""
    from .formats import gguf as G
    rng = np.random.default_rng(0)
    sizes = {G.GGML_Q4_0: (18, 32), G.GGML_Q8_0: (34, 32), G.GGML_Q2_K: (84, 256), G.GGML_Q3_K: (110, 256), G.GGML_Q4_K: (144, 256),
             G.GGML_Q5_K: (176, 256), G.GGML_Q6_K: (210, 256), G.GGML_IQ4_NL: (18, 32), G.GGML_IQ4_XS: (136, 256)}
    ok = True
    for kind, (bb, vals) in sizes.items():
        raw = rng.integers(0, 256, size=(4, bb), dtype=np.uint8)
        raw[:, :4] = np.frombuffer(np.full(8, 0.01, dtype="<f2").tobytes(), dtype=np.uint8).reshape(4, 4) if kind in (G.GGML_Q4_K, G.GGML_Q5_K) else raw[:, :4]
        half = np.frombuffer(np.float16(0.02).tobytes(), dtype=np.uint8)
        for off in {G.GGML_Q4_0: [0], G.GGML_Q8_0: [0], G.GGML_Q2_K: [80, 82], G.GGML_Q3_K: [108], G.GGML_Q4_K: [0, 2],
                    G.GGML_Q5_K: [0, 2], G.GGML_Q6_K: [208], G.GGML_IQ4_NL: [0], G.GGML_IQ4_XS: [0]}[kind]:
            raw[:, off : off + 2] = half
        v = G.decode(raw.reshape(-1), 0, 4 * vals, kind)
        ok &= v.shape == (4 * vals,) and bool(np.isfinite(v).all())
    return {"ok": ok, "types": len(sizes)}


def check_native_helpers() -> dict:
    """The C++ side: packed-row decode and GEMV oracle, split planner, prefix cache, slot book, expert-swap planner."""
    from . import formats as F
    from . import native
    from .quantize.nint import NintSpec, quantize_nint
    native.lib()  # raises with the build command when the shared object is missing
    w = _w(16, 256)
    t = quantize_nint(w, NintSpec(bits=4))
    rows = native.NintRows(np.frombuffer(F.pack_tensor(t)[1], dtype=np.uint8))
    x = np.random.default_rng(1).normal(size=256).astype(np.float32)
    dense = rows.decode()
    decode_ok = _rel_np(dense, F.dequantize(t)) < 1e-6 and _rel_np(rows.gemv(x), dense.astype(np.float64) @ x) < 1e-4
    plan = native.tp_plan(32, 4)
    plan_ok = [b - a for a, b in plan] == [8, 8, 8, 8] and plan[0][0] == 0 and plan[-1][1] == 32
    cache = native.PrefixCache(None, ram_budget=1 << 20, block_tokens=16)
    keys = cache.keys(list(range(64)))
    blob = np.arange(256, dtype=np.uint8)
    cache.put(keys[0], blob)
    got = cache.get(keys[0], blob.nbytes)
    cache_ok = got is not None and bytes(got) == bytes(blob) and cache.match(keys) == 1 and len(keys) == 4
    cache.close()
    book = native.SlotBook(2)
    s0, _ = book.acquire(10)
    s1, _ = book.acquire(11)
    _, evicted = book.acquire(12)
    book_ok = {s0, s1} == {0, 1} and evicted in (10, 11) and book.lookup(12) >= 0
    swaps = native.moe_rank_swaps([9.0, 1.0, 8.0, 0.5], [0, 1, 1, 0], 2)
    return {"ok": bool(decode_ok and plan_ok and cache_ok and book_ok and swaps == [(1, 0)]),
            "decode": bool(decode_ok), "plan": plan_ok, "prefix_cache": bool(cache_ok), "slot_book": bool(book_ok), "swaps": swaps}


def check_natscale() -> dict:
    from .calibration import natscale as ns
    g = np.exp(np.random.default_rng(0).normal(size=40) * 2)
    beta = ns.natscale_exponent(g, 1.0)
    sol = ns.allocate_hulls(np.array([10, 20, 40]), np.array([[3.0, 2.0, 1.0], [5.0, 1.0, 0.5], [2.0, 1.9, 1.8]]), 70)
    return {"ok": abs(ns.realized_contrast(g, beta) - 1.0) < 1e-6 and sol["bytes"] <= 70 and sol["lower_bound"] <= sol["objective"] + 1e-12,
            "beta": round(beta, 4), "choice": sol["choice"].tolist()}


def check_tensor_schema() -> dict:
    from .architectures import canonical_name, detect_family
    cases = {"model.layers.3.self_attn.q_proj.weight": "model.block.3.attention.query.weight",
             "model.language_model.layers.0.linear_attn.out_proj.weight": "model.block.0.linear_attention.output.weight",
             "model.layers.1.mlp.experts.7.down_proj.weight": "model.block.1.mlp.experts.down.weight",
             "mtp.fc.weight": "predictor.fusion.weight"}
    bad = {k: canonical_name(k) for k, want in cases.items() if (canonical_name(k) or (None,))[0] != want}
    fam = detect_family({"model_type": "qwen3_next"}) == "qwen3_next" and detect_family({"model_type": "deepseek_v3"}) == "deepseek_v3"
    return {"ok": not bad and fam, "mismatches": {k: str(v) for k, v in bad.items()}}


def check_mtp_policy() -> dict:
    from .engine.mtp_policy import CycleDepthController, verify_greedy
    ctl = CycleDepthController(3)
    seen = []
    for _ in range(12):
        d = ctl.next_depth()
        seen.append(d)
        ctl.observe(d, accepted=min(d, 1), cycle_ms=1.0 + 0.4 * d)
    acc, _tok = verify_greedy(torch.tensor([4, 5, 6]), torch.tensor([4, 5, 9, 1]))
    return {"ok": set(seen[:3]) == {1, 2, 3} and acc == 2 and all(1 <= d <= 3 for d in seen), "depths": seen}


def check_gdn_chunked() -> dict:
    """Chunked Gated DeltaNet prefill against the token-serial kernels on one problem."""
    from .ops import gdn
    dev, L, hk, hv, d = "cuda", 200, 2, 4, 128
    g = torch.Generator(device=dev).manual_seed(0)
    c = 2 * hk * d + hv * d
    qkv = torch.randn((L, c), device=dev, generator=g) * 0.5
    z = torch.randn((L, hv * d), device=dev, generator=g).to(torch.bfloat16)
    a = torch.randn((L, hv), device=dev, generator=g).to(torch.bfloat16)
    b = torch.randn((L, hv), device=dev, generator=g).to(torch.bfloat16)
    al, dt, nw = torch.randn(hv, device=dev, generator=g) * 0.5, torch.randn(hv, device=dev, generator=g) * 0.5, torch.ones(d, device=dev)
    slot = torch.zeros(1, dtype=torch.int32, device=dev)
    outs = []
    for chunked in (True, False):
        keep = gdn.CHUNKED_MIN_TOKENS
        gdn.CHUNKED_MIN_TOKENS = 64 if chunked else 1 << 30
        try:
            st = torch.zeros((1, hv, d, d), device=dev)
            y = gdn.recurrent(qkv.clone(), z, a, b, al, dt, nw, st, slot, L, hk, hv)
        finally:
            gdn.CHUNKED_MIN_TOKENS = keep
        outs.append((y.float(), st))
    err_y, err_s = _rel(outs[0][0], outs[1][0]), _rel(outs[0][1], outs[1][1])
    return {"ok": err_y < 2e-2 and err_s < 2e-3, "output_rel_err": err_y, "state_rel_err": err_s}


def check_packed_experts() -> dict:
    """Packed NINT experts: the grouped product that decodes in registers against the exact host reconstruction."""
    from .ops import moe as moe_ops
    from .ops import packed
    n_out, k_in, tokens, top_k = 128, 512, 12, 2
    pe = packed.PackedExperts.synthetic(4, n_out, k_in, [2, 3, 4, 16], "cuda", gs=32, seed=3, std=0.02)
    g = torch.Generator(device="cuda").manual_seed(5)
    x = torch.randn((tokens, k_in), generator=g, device="cuda").to(torch.bfloat16)
    ids = torch.stack([torch.randperm(4, generator=g, device="cuda")[:top_k] for _ in range(tokens)]).to(torch.int32)
    plan = moe_ops.plan_routes(ids, 0, 4, token_tile=16)
    got = packed.packed_gemv_grouped(pe, x, plan, gather=True)
    rows = int(plan.totals[0])
    offsets, src = plan.offsets.cpu().tolist(), plan.src_token.cpu().tolist()
    want = torch.zeros((rows, n_out), device="cuda")
    for e in range(4):
        w = pe.dense(e).float()
        for r in range(offsets[e], offsets[e + 1]):
            want[r] = w @ x[src[r]].float()
    err = _rel(got[:rows].float(), want)
    return {"ok": rows == tokens * top_k and err < 3e-2, "rows": rows, "max_rel_err": err,
            "bits_per_weight": round(pe.bits_per_weight(), 3)}


def check_mla_latent_cache() -> dict:
    """Latent-attention decode over the 576-wide shared-row cache against the fp32 restatement on the same pages."""
    from .engine.kv_cache import LayerKV, PagedKVCache
    from .ops import mla as mla_ops
    from .ops import reference as ref
    g = torch.Generator().manual_seed(0)
    lens = [1, 33, 150]
    b = len(lens)
    cache = PagedKVCache(layers=1, kv_heads=1, head_dim=mla_ops.ROW_WIDTH, num_pages=64, max_seqs=b, max_pages_per_seq=12, device="cuda")
    kv = cache.layer(0)
    for r, n in enumerate(lens):
        cache.assign(r, 900 + r, n)
        rows = (torch.randn((n, mla_ops.ROW_WIDTH), generator=g) * 0.7).to(torch.bfloat16).cuda()
        mla_ops.latent_write(rows, cache.slots(900 + r, 0, n).cuda(), kv)
    q = (torch.randn((b, 16, mla_ops.ROW_WIDTH), generator=g) * 0.3).to(torch.bfloat16).cuda()
    seq_lens = torch.tensor(lens, dtype=torch.int32, device="cuda")
    got = mla_ops.decode(q, kv, cache.block_table[:b], seq_lens, sm_scale=0.07, splits=2).float().cpu()
    host = LayerKV(kv.k.cpu(), kv.v.cpu(), kv.k_scale.cpu(), kv.v_scale.cpu(), kv.page_size)
    want = ref.paged_attn_decode(q.cpu(), host, cache.block_table[:b].cpu(), seq_lens.cpu(), 0.07, 1).float()[:, :, : mla_ops.LATENT]
    err = _rel(got, want)
    return {"ok": err < 2e-2, "max_rel_err": err, "bytes_per_token": cache.bytes_per_token()}


def check_moe_grouped() -> dict:
    """Router top-k, route plan, grouped FP8 expert GEMMs and combine against a per-expert fp32 loop."""
    from .ops import moe as moe_ops
    from .ops import reference as ref
    from .quantize.fp8_block import quantize_fp8_block_torch
    e, h, inter, t, k = 8, 512, 256, 24, 2
    g = torch.Generator(device="cuda").manual_seed(2)
    x = torch.randn((t, h), device="cuda", generator=g).to(torch.bfloat16)
    router = (torch.randn((e, h), device="cuda", generator=g) * 0.05).to(torch.bfloat16)
    ids, wt, scores = moe_ops.router_topk(x, router, k, want_scores=True)
    routed_ok = torch.equal(ids.long().sort(-1).values, scores.topk(k, -1).indices.sort(-1).values)
    gu_f = (torch.randn((e, 2 * inter, h), generator=g, device="cuda") * 0.05).to(torch.bfloat16)
    dn_f = (torch.randn((e, h, inter), generator=g, device="cuda") * 0.05).to(torch.bfloat16)
    gu_q, gu_s = (torch.stack(v) for v in zip(*[quantize_fp8_block_torch(m) for m in gu_f]))
    dn_q, dn_s = (torch.stack(v) for v in zip(*[quantize_fp8_block_torch(m) for m in dn_f]))
    xq, xs = ref.quant_rows(x)
    got = moe_ops.moe_ffn_fp8(xq, xs, ids, wt, gu_q, gu_s, dn_q, dn_s)
    want = torch.zeros((t, h), device="cuda")
    xd = xq.float() * xs[:, None]
    for le in range(e):
        tok, slot = (ids == le).nonzero(as_tuple=True)
        if tok.numel() == 0:
            continue
        gu = (xd[tok] @ ref.dequant_block(gu_q[le], gu_s[le]).T).to(torch.bfloat16)
        hq, hs = ref.silu_mul_quant(gu)
        y = ((hq.float() * hs[:, None]) @ ref.dequant_block(dn_q[le], dn_s[le]).T).to(torch.bfloat16).float()
        want.index_add_(0, tok, y * wt[tok, slot][:, None])
    err = float((got.float() - want).abs().mean() / (want.abs().mean() + 1e-12))  # single re-quantized codes may flip: compare means
    return {"ok": bool(routed_ok) and err < 2e-2, "routing_matches": bool(routed_ok), "mean_rel_err": err}


CPU_CHECKS = {"nint": check_nint_roundtrip, "fp8-block": check_fp8_block_roundtrip, "tp-linear": check_tp_linear,
              "ep-moe": check_ep_moe, "continuous-batching": check_continuous_batching, "json-constraint": check_json_constraint,
              "codecs": check_codecs, "mfe": check_mfe_and_expert_mix, "fp8-sq": check_fp8_sq_palettes, "gguf-blocks": check_gguf_blocks,
              "native": check_native_helpers, "natscale": check_natscale, "tensor-schema": check_tensor_schema,
              "mtp-policy": check_mtp_policy}
GPU_CHECKS = {"fp8-gemm": check_fp8_gemm, "attention": check_attention, "engine": check_engine_greedy, "gdn-chunked": check_gdn_chunked,
              "packed-experts": check_packed_experts, "mla-latent-cache": check_mla_latent_cache, "moe-grouped": check_moe_grouped}


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
    if getattr(args, "list", False):
        print(json.dumps({"anywhere": sorted(CPU_CHECKS) + ["container"], "gpu": sorted(GPU_CHECKS)}, indent=1))
        return 0
    report = run(args.check or None)
    print(json.dumps(report, indent=1))
    return 0 if report["ok"] else 1
