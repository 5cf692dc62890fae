"""Quality figures of the quantizers and of the FP8 GPU path, printed as one JSON object per measurement.

    python -m mfq_b200.evaluation.quality_report tiny-moe [--reference baseline/_ref]
    python -m mfq_b200.evaluation.quality_report fp8-llama [--device cuda]

``tiny-moe``: the tiny random-init mixture-of-experts model (2 layers, hidden 256, 8 experts top-2, vocabulary 1024) with
every expert projection quantized to NINT4, NVQ3 or MXFP4 by the seeded balanced allocation; KL divergence and top-1
agreement of the quantized model against the bf16 model over a 64-token prompt and 32 greedy tokens.  With
``--reference`` pointing at an installed copy of the reference package, the same weights and the same per-expert family
allocation are also quantized by the reference's own NumPy quantizers (``mfq/formats/nint.py: quantize``,
``mfq/quantize/nvq_quant.py: quantize``; MXFP4 experts use this repository's encoder in both arms, the reference has no
bf16 -> MXFP4 quantizer) and scored the same way.

``fp8-llama``: the block-FP8 Llama path (E4M3 weights with 128x128 multipliers, per-row E4M3 activations, FP8 KV pages)
against an fp32 evaluation of the SAME random-init weights before quantization (a small dense decoder, so the float
model is cheap), prefill logits of a 256-token prompt.  On ``cuda`` this exercises the hand-written kernels.
"""

from __future__ import annotations

import argparse
import json
import sys

import numpy as np
import torch

from .kld import compare_logits, teacher_forced_report


def tiny_moe(reference: str | None) -> list[dict]:
    from ..models.moe_lm import MoeConfig, MoeLM, dequantize_checkpoint, init_weights, quantize_moe_checkpoint
    from ..quantize.expertwise import balanced_expert_mix, parse_profiles
    cfg = MoeConfig()
    w = init_weights(cfg, seed=0)
    mix, seed = "NINT4,NVQ3,MXFP4", 20260908
    prompt = torch.randint(0, cfg.vocab_size, (64,), generator=torch.Generator().manual_seed(1))
    out = []
    ours = dequantize_checkpoint(quantize_moe_checkpoint(w, mix, seed=seed))
    rep, _ = teacher_forced_report(MoeLM(cfg, w), MoeLM(cfg, ours), prompt, 32)
    out.append({"case": "tiny-moe", "quantizers": "this repository", "mix": mix, **rep.as_dict()})
    if reference:
        sys.path.insert(0, reference)
        from mfq.formats import nint as rnint  # type: ignore
        from mfq.formats.nvq import NvqSpec as RNvqSpec  # type: ignore
        from mfq.quantize import nvq_quant as rnvq  # type: ignore
        from ..formats import dequantize as our_dequantize
        from ..quantize.mxfp4 import quantize_mxfp4
        profiles = parse_profiles(mix)
        ref_w = {}
        for name, t in w.items():
            a = t.numpy().astype(np.float32)
            if ".mlp.experts." not in name or a.ndim != 3:
                ref_w[name] = torch.from_numpy(a).to(torch.bfloat16).float()
                continue
            assign = balanced_expert_mix(name, a.shape[0], len(profiles), seed)
            rec = np.empty_like(a)
            for e in range(a.shape[0]):
                prof = profiles[int(assign[e])]
                if prof.nint is not None:
                    spec = rnint.NintSpec(bits=prof.nint.bits, groupsize=prof.nint.groupsize, sub_bits=prof.nint.sub_bits)
                    rec[e] = np.stack([rnint.dequantize(rnint.quantize(row, spec)) for row in a[e]])
                elif prof.nvq is not None:
                    spec = RNvqSpec(codebook=prof.nvq.codebook, groupsize=prof.nvq.groupsize, sub_bits=prof.nvq.sub_bits)
                    rec[e] = rnvq.dequantize(rnvq.quantize(a[e], spec))
                else:
                    rec[e] = our_dequantize(quantize_mxfp4(a[e]))
            ref_w[name] = torch.from_numpy(rec)
        rep, _ = teacher_forced_report(MoeLM(cfg, w), MoeLM(cfg, ref_w), prompt, 32)
        out.append({"case": "tiny-moe", "quantizers": "reference NumPy (NINT, NVQ) + this repository (MXFP4)", "mix": mix,
                    **rep.as_dict()})
    return out


def _float_llama_logits(cfg, t: dict, ids: torch.Tensor) -> torch.Tensor:
    """fp32 forward of the dense decoder over float weights (causal attention over the whole prompt)."""
    h = t["embed"][ids.long()].float()
    n, d, hq, hk = ids.numel(), cfg.head_dim, cfg.num_heads, cfg.num_kv_heads
    pos = torch.arange(n, dtype=torch.float32)
    inv = torch.exp2(-np.log2(cfg.rope_theta) * (2 * torch.arange(d // 2, dtype=torch.float32)) / d)
    ang = pos[:, None] * inv[None]
    cos, sin = ang.cos()[:, None], ang.sin()[:, None]

    def rms(x, w):
        return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + cfg.rms_eps) * w.float()

    def rope(x):
        a, b = x[..., : d // 2], x[..., d // 2 :]
        return torch.cat([a * cos - b * sin, b * cos + a * sin], -1)

    mask = torch.full((n, n), float("-inf")).triu(1)
    for l in t["layers"]:
        x = rms(h, l["attn_norm"])
        q = rope((x @ l["wq"].float().T).view(n, hq, d))
        k = rope((x @ l["wk"].float().T).view(n, hk, d))
        v = (x @ l["wv"].float().T).view(n, hk, d)
        k, v = k.repeat_interleave(hq // hk, 1), v.repeat_interleave(hq // hk, 1)
        s = torch.einsum("qhd,khd->hqk", q, k) / np.sqrt(d) + mask
        o = torch.einsum("hqk,khd->qhd", torch.softmax(s, -1), v).reshape(n, hq * d)
        h = h + o @ l["wo"].float().T
        x = rms(h, l["mlp_norm"])
        h = h + (torch.nn.functional.silu(x @ l["wg"].float().T) * (x @ l["wu"].float().T)) @ l["wd"].float().T
    return rms(h, t["final_norm"]) @ t["head"].float().T


def fp8_llama(device: str) -> list[dict]:
    from ..engine.llm_engine import LLMEngine
    from ..models.llama import Fp8Linear, LlamaConfig, LlamaLayer, LlamaModel, LlamaWeights, StepBuffers
    cfg = LlamaConfig(vocab_size=4096, hidden_size=512, intermediate_size=1536, num_layers=4, num_heads=4, num_kv_heads=2,
                      head_dim=128, rope_theta=1e4, name="llama-small-fp8")
    g = torch.Generator().manual_seed(0)
    h, i, d = cfg.hidden_size, cfg.intermediate_size, cfg.head_dim

    def rnd(r, c, std=0.04):
        return (torch.randn((r, c), generator=g) * std).to(torch.bfloat16)
    ft = {"embed": rnd(cfg.vocab_size, h, 1.0), "head": rnd(cfg.vocab_size, h), "final_norm": torch.ones(h, dtype=torch.bfloat16), "layers": []}
    layers = []
    dev = torch.device(device)
    for _ in range(cfg.num_layers):
        l = {"attn_norm": torch.ones(h, dtype=torch.bfloat16), "mlp_norm": torch.ones(h, dtype=torch.bfloat16),
             "wq": rnd(cfg.num_heads * d, h), "wk": rnd(cfg.num_kv_heads * d, h), "wv": rnd(cfg.num_kv_heads * d, h),
             "wo": rnd(h, cfg.num_heads * d), "wg": rnd(i, h), "wu": rnd(i, h), "wd": rnd(h, i)}
        ft["layers"].append(l)
        layers.append(LlamaLayer(attn_norm=l["attn_norm"].to(dev), qkv=Fp8Linear.from_float(torch.cat([l["wq"], l["wk"], l["wv"]], 0).to(dev)),
                                 o_proj=Fp8Linear.from_float(l["wo"].to(dev)), mlp_norm=l["mlp_norm"].to(dev),
                                 gate_up=Fp8Linear.from_float(torch.cat([l["wg"], l["wu"]], 0).to(dev)), down=Fp8Linear.from_float(l["wd"].to(dev))))
    w = LlamaWeights(ft["embed"].to(dev), layers, ft["final_norm"].to(dev), Fp8Linear.from_float(ft["head"].to(dev)))
    model = LlamaModel(cfg, w)
    n = 256
    ids = torch.randint(0, cfg.vocab_size, (n,), generator=torch.Generator().manual_seed(3))
    eng = LLMEngine(model, max_batch=1, max_seq_len=n + 16, device=dev, use_graphs=False)
    eng.cache.assign(0, 0, n)
    step = StepBuffers(input_ids=ids.to(dev, torch.int32), positions=torch.arange(n, dtype=torch.int32, device=dev),
                       slots=eng.cache.slots(0, 0, n).to(dev), cu_seqlens=[0, n])
    got = model.forward(step, eng.cache, prefill=True).float().cpu()
    rep = compare_logits(_float_llama_logits(cfg, ft, ids), got)
    return [{"case": "fp8-llama", "device": device, "model": "4 layers, hidden 512, vocabulary 4096, random-init N(0, 0.04)",
             "baseline": "fp32 evaluation of the unquantized weights", **rep.as_dict()}]


def main(argv=None) -> None:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("case", choices=["tiny-moe", "fp8-llama"])
    ap.add_argument("--reference", default=None, help="directory that holds the installed reference package (its parent of `mfq/`)")
    ap.add_argument("--device", default="cpu")
    args = ap.parse_args(argv)
    rows = tiny_moe(args.reference) if args.case == "tiny-moe" else fp8_llama(args.device)
    for r in rows:
        print(json.dumps({k: (round(v, 6) if isinstance(v, float) else v) for k, v in r.items()}))


if __name__ == "__main__":
    main()
