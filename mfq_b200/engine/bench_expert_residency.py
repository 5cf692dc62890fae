"""Decode throughput of a small MoE decoder whose routed experts sit behind an HBM slot arena: eager wave-by-wave
decoding against decoding inside CUDA graphs with device-side slot translation and miss replay.

    python -m mfq_b200.engine.bench_expert_residency [--slots 6] [--rows 4] [--tokens 200]

Prints one JSON line: total device time of ``--tokens`` decode steps per mode (CUDA events around ``generate``, after a
16-token warm-up run), the graph mode's replay / wave-fallback counts and the uploads of both.
"""

from __future__ import annotations

import argparse
import json

import torch


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--slots", type=int, default=6, help="arena slots per layer (the tiny decoder has 8 experts)")
    ap.add_argument("--rows", type=int, default=4)
    ap.add_argument("--tokens", type=int, default=200)
    args = ap.parse_args(argv)
    from ..models.moe_decoder import MoeDecoderConfig, MoeDecoderModel, MoeWeights
    from ..models.moe_lm import MoeConfig, init_weights
    from .llm_engine import LLMEngine
    cfg = MoeDecoderConfig.tiny()
    tensors = init_weights(MoeConfig(head_dim=128, hidden_size=256, moe_intermediate=128, shared_intermediate=128), seed=4, std=0.05)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=torch.Generator().manual_seed(n)) for n in (17, 40, 23, 31, 19, 45, 28, 36)[: args.rows]]
    out = {"slots": args.slots, "rows": len(prompts), "tokens_per_row": args.tokens}
    for name, graphs in (("eager_waves", False), ("graphs_optimistic", True)):
        eng = LLMEngine(MoeDecoderModel(cfg, MoeWeights.from_tensors(cfg, tensors, "cuda", expert_slots=args.slots)),
                        max_batch=len(prompts), max_seq_len=max(512, args.tokens + 64), use_graphs=graphs)
        if graphs and not eng.enable_expert_residency_graphs():
            raise SystemExit("this engine cannot decode an expert arena inside graphs")
        eng.generate(prompts, 16)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        r = eng.generate(prompts, args.tokens)
        e1.record()
        torch.cuda.synchronize()
        out[name] = {"ms_total": round(e0.elapsed_time(e1), 2), "tokens": int(r.tokens.numel()),
                     "stats": getattr(eng, "residency_stats", None), "uploads": sum(x.stats["uploads"] for x in eng.model.residencies())}
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
