"""Flagship benchmark: Llama-style 8B in block-scaled FP8, FP8 paged KV (16-token pages), greedy decode.

    python bench.py --gpus 1 --steps 64 --warmup 4
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        bench.py --gpus N --steps K --warmup W          # ONE model tensor-parallel over the N GPUs, global batch 64
                                                        # (strong scaling); --parallelism dp runs N replicas instead
    python bench.py --impl reference ...                # the unmodified reference, when it is available

A step is one decode step of a batch of 64 sequences, each with a 4096-token context (prefilled by the
engine, outside the timed region).  Reported: aggregate decode tokens/s at batch 64 (``value``), and in
``extra`` single-stream decode tokens/s and prefill tokens/s of one 4096-token prompt.  Device timing uses CUDA
events around exactly ``steps`` graph replays, bracketed by barrier + synchronize, max over ranks.  The
``e2e`` figure drives the same steps through ``LLMEngine.step_host``: every step copies that step's input ids
from pinned host memory to the device and reads the sampled ids back to the host.

Weights are random N(0, 0.02) quantized to E4M3 with 128x128 fp32 multipliers; prompts are uniform random ids.
Every timed step streams the full weight set (>= 8 GB, far beyond the 126 MB L2), so no L2 flush is needed.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

PUBLISHED_BATCHED_DECODE_TOK_S = 156.56  # reference: continuous batching 32 x 256 tokens, graph replay, RTX 3090 Ti
PUBLISHED_SINGLE_DECODE_TOK_S = 87.0  # reference headline: single-stream MTP decode, RTX 3090 Ti


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int) -> None:
        self.index, self.rows, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-i", str(self.index), "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *exc):
        if self.proc is not None:
            time.sleep(0.15)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self) -> dict:
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
            except (ValueError, IndexError):
                continue
            for name, flag in zip(names, r[3:7]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def run_ours(args) -> dict:
    import torch
    import torch.distributed as dist

    from mfq_b200 import ops
    from mfq_b200.engine.llm_engine import LLMEngine
    from mfq_b200.models.llama import LlamaConfig, LlamaModel, LlamaWeights

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run for N > 1")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    collective = None
    tp = world if args.parallelism == "tp" else 1  # dp: every GPU serves its own replica and its own batch
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
        if tp > 1:
            from mfq_b200.parallel.tensor_parallel import TensorParallel
            collective = TensorParallel(dist.group.WORLD, dev)

    cfg = LlamaConfig.tiny() if args.tiny else LlamaConfig.llama_8b()
    batch, ctx, new = args.batch, args.context, args.steps + args.warmup + 8
    weights = LlamaWeights.random_init(cfg, dev, seed=0, tp_rank=rank if tp > 1 else 0, tp_size=tp, weight_format=args.weights)
    model = LlamaModel(cfg, weights, collective=collective)
    engine = LLMEngine(model, max_batch=batch, max_seq_len=ctx + 2 * new + 16)
    ops.count_launches(True)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def phase(name: str) -> None:  # progress on stderr: a run that stops shows where
        if rank == 0:
            print(f"[bench] {name} t={time.time() - t_start:.1f}s", file=sys.stderr, flush=True)
    t_start = time.time()

    def max_over_ranks(ms: float) -> float:
        if world == 1:
            return ms
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    replicas = world // tp  # independent serving replicas; the job's throughput is the sum over them
    gen = torch.Generator().manual_seed(1234 + (rank if tp == 1 else 0))
    prompts = [torch.randint(0, cfg.vocab_size, (ctx,), generator=gen) for _ in range(batch)]

    # ---- prefill: warm once on row 0, time one 4096-token prompt, then fill every row ----
    phase("weights ready")
    engine.prefill(0, prompts[0])
    barrier()
    phase("first prefill done")
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    engine.prefill(0, prompts[0])
    e1.record()
    barrier()
    prefill_ms = max_over_ranks(e0.elapsed_time(e1))
    for row in range(batch):
        if row:
            engine.prefill(row, prompts[row])
        engine.grow(row, ctx + 2 * new + 8)
    barrier()
    ops.Workspace.get(dev).check()
    phase("all rows prefilled")

    def timed_decode(b: int, steps: int, warmup: int):
        for _ in range(warmup):
            engine.decode_step(b)
        barrier()
        launches0 = ops.launch_count()
        a, z = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with ClockSampler(local) as clocks:
            a.record()
            for _ in range(steps):
                engine.decode_step(b)
            z.record()
            barrier()
        return max_over_ranks(a.elapsed_time(z)), clocks.summary()

    ms64, clocks = timed_decode(batch, args.steps, args.warmup)
    ops.Workspace.get(dev).check()
    phase("batched decode timed")
    if args.profile_steps:  # a profiler started with its collection off sees exactly these steps
        torch.cuda.synchronize()
        torch.cuda.profiler.start()
        for _ in range(args.profile_steps):
            engine.decode_step(batch)
        torch.cuda.synchronize()
        torch.cuda.profiler.stop()
    launches = engine.launches_per_step.get(batch, 0) * args.steps
    ms1, _ = timed_decode(1, args.steps, args.warmup)
    ops.Workspace.get(dev).check()
    phase("single-stream decode timed")
    ms32 = None
    if batch >= 32:  # the reference accepts at most 32 concurrent sequences: one pair of figures at the same batch
        ms32, _ = timed_decode(32, args.steps, args.warmup)
    engine_launches = dict(engine.launches_per_step)

    # ---- end to end through the public step API: pinned H2D of the inputs + D2H of the result every step ----
    host_in = torch.zeros(batch, dtype=torch.int32).pin_memory()
    host_out = torch.zeros(batch, dtype=torch.int32).pin_memory()
    host_in.copy_(engine.sampled[:batch].cpu())
    for _ in range(args.warmup):
        engine.step_host(host_in, host_out)
        host_in.copy_(host_out)
    barrier()
    a, z = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(args.steps):
        engine.step_host(host_in, host_out)
        host_in.copy_(host_out)
    z.record()
    barrier()
    e2e_ms = max_over_ranks(a.elapsed_time(z))
    ops.Workspace.get(dev).check()
    phase("end-to-end timed")

    # ---- the same tensor-parallel model with library collectives (unfused GEMM + NCCL all-reduce), for comparison ----
    nccl = {}
    if tp > 1 and args.nccl_baseline:
        try:
            from mfq_b200.parallel.tensor_parallel import NcclTensorParallel
            del engine
            torch.cuda.empty_cache()
            # eager launches: library collectives are kept out of CUDA-graph capture here
            base = LLMEngine(LlamaModel(cfg, weights, collective=NcclTensorParallel(dist.group.WORLD, dev)), max_batch=batch,
                             max_seq_len=ctx + 2 * new + 16, use_graphs=False)
            phase("library-collective engine built")
            for row in range(batch):
                base.prefill(row, prompts[row][: min(ctx, 512)])  # timing only: a short context fills the rows faster
                base.grow(row, ctx + 2 * new + 8)
            base.seq_lens[:batch] = ctx  # decode against full-length contexts (whatever the pages hold)
            for r in range(batch):
                base.row_len[r] = ctx
            engine = base
            n64, _ = timed_decode(batch, args.steps, args.warmup)
            n1, _ = timed_decode(1, args.steps, args.warmup)
            nccl = {"nccl_baseline_decode_tok_s_bs64": round(batch * args.steps / (n64 / 1e3), 2),
                    "nccl_baseline_decode_tok_s_bs1": round(args.steps / (n1 / 1e3), 2),
                    "nccl_baseline_note": "same model and kernels, row-parallel sums through ncclAllReduce after an unfused "
                                          "GEMM, eager launches (no CUDA graph)"}
        except Exception as exc:  # the comparison is optional: report why it is missing
            nccl = {"nccl_baseline_error": repr(exc)[:200]}

    value = replicas * batch * args.steps / (ms64 / 1e3)
    result = {
        "metric": "decode_tok_s_bs64", "value": round(value, 2), "unit": "tok/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(ms64 / args.steps, 4), "higher_is_better": True,
        "scaling": "strong" if tp > 1 else "weak",
        "vs_baseline": None, "dtype": "fp8_e4m3 weights/activations/KV, bf16 residual stream, fp32 accumulate",
        "data": "synthetic (uniform random token ids, random-init N(0,0.02) weights)", "impl": "ours",
        "config": {"model": cfg.name, "params_b": round(cfg.param_count() / 1e9, 2), "global_batch": batch * replicas, "seq_len": ctx,
                   "parallelism": f"tp{world}" if tp > 1 else f"dp{world}", "per_gpu_batch": batch if tp == 1 else None, "kv": "fp8 paged, 16-token pages", "weights": "E4M3, 128x128 fp32 block scales" if args.weights == "fp8" else
                   "4-bit codes + bf16 (scale, min) per 32 inputs, decoded inside the GEMM pipeline (LM head: E4M3)",
                   "l2": "inputs larger than L2 (every step streams all weights)"},
        "clocks": clocks,
        "e2e": {"value": round(replicas * batch * args.steps / (e2e_ms / 1e3), 2), "unit": "tok/s",
                "h2d_bytes_per_step": batch * 4 * replicas, "d2h_bytes_per_step": batch * 4 * replicas},
        "gpu_launches": launches * replicas,
        "extra": {"decode_tok_s_bs1": round(replicas * args.steps / (ms1 / 1e3), 2), "ms_per_step_bs1": round(ms1 / args.steps, 4),
                  "prefill_tok_s": round(replicas * ctx / (prefill_ms / 1e3), 1), "prefill_ms": round(prefill_ms, 2),
                  "decode_tok_s_bs32": round(replicas * 32 * args.steps / (ms32 / 1e3), 2) if ms32 else None,
                  "launches_per_step_bs64": engine_launches.get(batch), "launches_per_step_bs1": engine_launches.get(1),
                  "vs_published_bs64": round(value / PUBLISHED_BATCHED_DECODE_TOK_S, 2),
                  "vs_published_bs1": round(args.steps / (ms1 / 1e3) / PUBLISHED_SINGLE_DECODE_TOK_S, 2),
                  "published_note": "the reference publishes no number for this model or hardware (vs_baseline is null); the two "
                                    "ratios above divide by its 156.56 tok/s continuous batching and 87.0 tok/s headline, "
                                    "measured on one RTX 3090 Ti with a different model", **nccl},
    }
    if world > 1:
        dist.destroy_process_group()
    return result if rank == 0 else {}


def run_hybrid(args) -> dict:
    """Second model family (one GPU): the Qwen3-Next-style 80B-total / 3B-active hybrid -- 36 Gated-DeltaNet layers,
    12 gated-attention layers with 256-wide heads, 512 routed experts (top 10) + a shared expert per layer, an MTP
    draft head -- all weights in block FP8 (about 80 GB).  Reports prefill of one prompt, single-stream decode without
    and with draft/verify cycles, and batched decode."""
    import torch

    from mfq_b200 import ops
    from mfq_b200.engine.llm_engine import LLMEngine
    from mfq_b200.models.hybrid import HybridConfig, HybridModel, random_hybrid_weights

    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run for N > 1")
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    collective = None
    if world > 1:  # one model over the GPUs: heads tensor-parallel, experts split over the ranks
        from mfq_b200.parallel.tensor_parallel import TensorParallel
        dist.init_process_group("nccl", device_id=dev)
        collective = TensorParallel(dist.group.WORLD, dev)
    cfg = HybridConfig.tiny() if args.tiny else HybridConfig.next_80b()
    batch, ctx, new = args.batch, args.context, args.steps + args.warmup + 8
    use_mtp = world == 1  # draft/verify cycles are measured on one GPU only
    t0 = time.time()
    weights = random_hybrid_weights(cfg, dev, seed=0, mtp=use_mtp, tp_rank=rank, tp_size=world,
                                    expert_format="packed" if args.weights == "packed" else "fp8")
    torch.cuda.synchronize()
    build_s = time.time() - t0
    engine = LLMEngine(HybridModel(cfg, weights, collective=collective), max_batch=batch, max_seq_len=ctx + 4 * new + 16,
                       mtp_draft_tokens=1 if use_mtp else 0)

    def sync():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms: float) -> float:
        if world == 1:
            return ms
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())
    gen = torch.Generator().manual_seed(1234)
    prompts = [torch.randint(0, cfg.vocab_size, (ctx,), generator=gen) for _ in range(batch)]

    def timed(fn, steps, warmup):
        for _ in range(warmup):
            fn()
        sync()
        a, z = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with ClockSampler(local) as clocks:
            a.record()
            for _ in range(steps):
                fn()
            z.record()
            sync()
        return max_over_ranks(a.elapsed_time(z)), clocks.summary()

    engine.prefill(0, prompts[0])
    sync()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    engine.prefill(0, prompts[0])
    e1.record()
    sync()
    prefill_ms = max_over_ranks(e0.elapsed_time(e1))
    for row in range(batch):
        if row:
            engine.prefill(row, prompts[row])
        engine.grow(row, ctx + 4 * new + 8)
    engine.active.fill_(1)
    torch.cuda.synchronize()
    ops.Workspace.get(dev).check()
    ms64, clocks = timed(lambda: engine.decode_step(batch), args.steps, args.warmup)
    ms1, _ = timed(lambda: engine.decode_step(1), args.steps, args.warmup)
    ms1_mtp = ms64_mtp = float("nan")
    stats = {}
    if use_mtp:
        ms1_mtp, _ = timed(lambda: engine.mtp_step(1), args.steps, args.warmup)
        stats = engine.mtp_stats()
        ms64_mtp, _ = timed(lambda: engine.mtp_step(batch), args.steps, args.warmup)
    sync()
    ops.Workspace.get(dev).check()
    value = batch * args.steps / (ms64 / 1e3)
    num = lambda v, nd=4: None if v != v else round(v, nd)  # NaN (not measured at this N) -> null
    result = {
        "metric": "decode_tok_s_bs64", "value": round(value, 2), "unit": "tok/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(ms64 / args.steps, 4), "higher_is_better": True,
        "scaling": "strong" if world > 1 else "weak",
        "vs_baseline": None,
        "dtype": "fp8_e4m3 weights/activations/KV, bf16 residual stream, fp32 accumulate and recurrent state",
        "data": "synthetic (uniform random token ids, random-init N(0,0.02) weights)", "impl": "ours",
        "config": {"model": cfg.name, "global_batch": batch, "seq_len": ctx, "parallelism": f"tp{world}+ep{world}" if world > 1 else "dp1",
                   "weights_gb": round(weights.nbytes() / 1e9, 1) if hasattr(weights, "nbytes") else None,
                   "experts": "packed NINT2-5 / MXFP4 mix, decoded in registers" if args.weights == "packed" else "block FP8",
                   "l2": "inputs larger than L2 (the routed experts of a step alone exceed it)"},
        "clocks": clocks,
        "extra": {"decode_tok_s_bs1": round(args.steps / (ms1 / 1e3), 2), "ms_per_step_bs1": round(ms1 / args.steps, 4),
                  "mtp_cycle_ms_bs1": num(ms1_mtp / args.steps), "mtp_cycle_ms_bs64": num(ms64_mtp / args.steps),
                  "mtp_acceptance_random_head": stats.get("acceptance_rate"),
                  "mtp_note": "one draft token per cycle; a random-init draft head is never accepted, so a cycle yields one "
                              "token here -- at the reference's published 88% acceptance a cycle yields 1.88",
                  "decode_tok_s_bs1_mtp_at_88pct": num(1.88 * args.steps / (ms1_mtp / 1e3), 2),
                  "prefill_tok_s": round(ctx / (prefill_ms / 1e3), 1), "prefill_ms": round(prefill_ms, 2),
                  "weight_build_s": round(build_s, 1),
                  "vs_baseline_bs1": round(args.steps / (ms1 / 1e3) / 62.9, 2),
                  "vs_baseline_prefill": round(ctx / (prefill_ms / 1e3) / 1779.7, 2),
                  "baseline_note": "reference: same model family (V1-S tier) on one RTX 3090 Ti + 32 GiB host RAM: prefill 1,779.7, "
                                   "decode 62.9, MTP decode 87.0 tok/s; continuous batching 156.56 tok/s"},
    }
    if world > 1:
        dist.destroy_process_group()
    return result if rank == 0 else {}


def run_reference(args) -> dict:
    from baseline import reference_arm
    return reference_arm.run(args)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--parallelism", choices=["dp", "tp"], default="tp",
                    help="N > 1: tp = one model sharded over the GPUs with the collectives fused into the kernels, global "
                         "batch fixed (strong scaling); dp = one replica per GPU, batch per GPU fixed (weak scaling)")
    ap.add_argument("--nccl-baseline", action="store_true",
                    help="tp: also time the same model with library (NCCL) collectives after unfused GEMMs (under extra)")
    ap.add_argument("--weights", choices=["fp8", "w4", "packed"], default="fp8",
                    help="block linears in block-scaled FP8 (default) or in the 4-bit NINT-native format (single GPU); "
                         "hybrid80b: 'packed' keeps the routed experts in a seeded mix of packed NINT 2-5 bit / MXFP4 "
                         "codes (about 3.4 bits per weight) decoded inside the expert kernels")
    ap.add_argument("--profile-steps", type=int, default=0,
                    help="after the timed region, run this many batched decode steps between cudaProfilerStart/Stop")
    ap.add_argument("--tiny", action="store_true", help="tiny model, for checking the harness itself")
    ap.add_argument("--model", choices=["llama8b", "hybrid80b"], default="llama8b",
                    help="llama8b: the flagship; hybrid80b: the Gated-DeltaNet + MoE hybrid with an MTP head (one GPU)")
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3
    if args.impl == "reference":
        out = run_reference(args)
    else:
        out = run_hybrid(args) if args.model == "hybrid80b" else run_ours(args)
    if out:
        print(json.dumps(out), flush=True)


if __name__ == "__main__":
    main()
