"""``mfq`` command line: build | quantize | inspect | eval | serve | bench.

The sub-commands and their main flags follow the reference CLI (``mfq/cli.py:660-741``, ``docs/cli/*.md``):
``mfq quantize <in> <out.mfq>`` with ``--bits/--groupsize/--sub-bits``, ``--preset``, ``--random-expert-mix`` +
``--random-expert-mix-seed``, ``--full-precision``, ``--split-max-size``, ``--device``, ``--dry-run``, ``--overwrite``;
``mfq serve --model ...`` with ``--host/--port/--api-key-env/--continuous-batching/--ctx-size/--tensor-parallel``;
``mfq eval kl`` for KLD / top-1 agreement; ``mfq build`` compiles the CUDA library.
"""

from __future__ import annotations

import argparse
import json

import numpy as np
import os
import sys
from pathlib import Path


def _cmd_build(args) -> int:
    from .ops.build import build
    path = build(force=args.force, verbose=args.verbose)
    manifest = {"backend": "cuda", "arch": "sm_100a", "library": str(path)}
    Path(args.manifest).parent.mkdir(parents=True, exist_ok=True)
    Path(args.manifest).write_text(json.dumps(manifest, indent=1))
    print(json.dumps(manifest))
    return 0


_SYNTHETIC = {
    "tiny-moe": dict(vocab_size=1024, hidden_size=256, num_layers=2, num_heads=4, num_kv_heads=2, head_dim=64,
                     rope_theta=1e6, rms_eps=1e-6, num_experts=8, top_k=2, moe_intermediate=128),
    "tiny-moe-128": dict(vocab_size=1024, hidden_size=256, num_layers=2, num_heads=4, num_kv_heads=2, head_dim=128,
                         rope_theta=1e6, rms_eps=1e-6, num_experts=8, top_k=2, moe_intermediate=128, shared_intermediate=128),
}


def _load_source(args):
    """-> (config dict, canonical float tensors, assets)."""
    import numpy as np
    src = args.input
    if src.startswith("synthetic:"):
        from .models.moe_lm import MoeConfig, init_weights
        kw = _SYNTHETIC[src.split(":", 1)[1]]
        w = init_weights(MoeConfig(**kw), seed=args.seed)
        return dict(kw, name=src), {k: v.numpy().astype(np.float32) for k, v in w.items()}, {}
    p = Path(src)
    if p.is_dir():
        from .checkpoint import read_hf_directory
        return read_hf_directory(p)
    if p.suffix == ".gguf":
        from .formats.gguf import read_gguf
        return read_gguf(p)
    if p.suffix == ".mfq":
        from . import formats as F
        with F.open_mfq(p) as store:
            assets = store.assets()
            cfg = json.loads(assets.pop("model_config.json"))
            tensors = {n: np.asarray(F.dequantize(store[n]), dtype=np.float32) for n in store if not n.startswith("__mfq_asset__/")}
        return cfg, tensors, assets
    raise SystemExit(f"cannot detect the source type of {src!r} (expected a Hugging Face directory, a .gguf file, an .mfq file or synthetic:<name>)")


def _cmd_quantize(args) -> int:
    from . import formats as F
    from .checkpoint import quantize_tensors, save_checkpoint
    out = Path(args.output)
    if out.exists() and args.resume_completed and not args.dry_run:
        try:  # a finished output from an earlier run: nothing to do
            with F.open_mfq(out) as done:
                n = sum(1 for k in done if not k.startswith("__mfq_asset__/"))
            print(json.dumps({"output": str(out), "already_complete": True, "tensors": n}))
            return 0
        except Exception:
            pass  # unreadable (cut short): quantize again over it
    elif out.exists() and not args.overwrite and not args.dry_run:
        raise SystemExit(f"{out} exists (use --overwrite)")
    cfg, tensors, assets = _load_source(args)
    base_records = None
    if args.base_mfq:
        # add a multi-token-prediction head to an existing checkpoint: everything the base holds is carried over as it is
        # (no re-quantization), only the source's predictor.* tensors are quantized and added
        with F.open_mfq(args.base_mfq) as base:
            base_records = {n: base[n] for n in base if not n.startswith("__mfq_asset__/")}
            base_assets = base.assets()
            cfg = json.loads(base_assets.pop("model_config.json"))
            base_assets.pop("model_graph.json", None)
            assets = {**base_assets, **assets}
        tensors = {n: t for n, t in tensors.items() if n.startswith("predictor.")}
        if not tensors:
            raise SystemExit(f"{args.input} has no multi-token-prediction head (predictor.* / mtp.* tensors) to add")
    dense = "bf16" if args.full_precision else (args.format or f"nint{args.bits}")
    widths = None
    if args.preset:
        from .quantize import presets
        preset = presets.normalize_preset(args.preset)
        dense = f"nint{presets.PRESETS[preset]}"
        topo = presets.Topology(int(cfg.get("num_layers", 0)), int(cfg.get("num_heads", 1)), int(cfg.get("num_kv_heads", 1)))
        widths = presets.plan(preset, {n: tuple(t.shape) for n, t in tensors.items()}, topo)
    if args.recipe:
        from .quantize.recipe import load_recipe
        widths = dict(widths or {})
        widths.update(load_recipe(args.recipe, list(tensors)))
    if args.target_bpw:
        widths = dict(widths or {})
        widths.update(_alphaq_widths(tensors, args.target_bpw))
    imatrix = scheme = None
    if args.imatrix:
        from .calibration.imatrix import load as load_imatrix
        imatrix = load_imatrix(args.imatrix)
    if args.ew_scheme:
        scheme = json.loads(Path(args.ew_scheme).read_text())
    row_widths = json.loads(Path(args.row_widths).read_text()) if getattr(args, "row_widths", None) else None
    def _label(n, t):
        if ".mlp.experts." in n and t.ndim == 3 and (args.random_expert_mix or scheme or dense != "bf16"):
            return "MFE"
        if widths is not None and n in widths:
            return "bf16" if widths[n] is None else f"nint{widths[n]}"
        return dense
    plan = {n: (list(t.shape), _label(n, t)) for n, t in tensors.items()}
    if args.dry_run:
        print(json.dumps({"tensors": len(plan), "dense": dense, "expert_mix": args.random_expert_mix, "plan": plan}, indent=1))
        return 0
    if dense.startswith("nint") and (args.groupsize or args.sub_bits):
        from .quantize import expertwise
        bits = int(dense[4:])
        gs, k = expertwise._NINT_PRESETS[bits]
        expertwise._NINT_PRESETS[bits] = (args.groupsize or gs, args.sub_bits or k)
    store = None
    if not args.no_temp and not args.fp8_sq_bits and not args.mxfp4_sq_bits and row_widths is None:
        from .quantize.resume import ResumeStore
        store = ResumeStore(str(out) + ".tmp", resume=args.resume, keep=args.keep_temp)
    q = quantize_tensors(tensors, dense=dense, expert_mix=args.random_expert_mix, seed=args.random_expert_mix_seed,
                         widths=widths, imatrix=imatrix, scheme=scheme, device=args.device, resume=store,
                         fp8_sq_bits=args.fp8_sq_bits, row_widths=row_widths, mxfp4_sq_bits=args.mxfp4_sq_bits,
                         progress=(lambda n: print(f"quantize {n}", file=sys.stderr)) if args.verbose else None)
    extra = {"quantization": {"dense": dense, "preset": args.preset or None, "imatrix": bool(imatrix), "ew_scheme": bool(scheme), "random_expert_mix": args.random_expert_mix.split(",") if args.random_expert_mix else [],
                              "random_expert_mix_seed": args.random_expert_mix_seed if args.random_expert_mix else None}}
    from .formats import runtime_profile as rp
    inherited = None
    if str(args.input).endswith(".mfq") and Path(args.input).is_file():
        with F.open_mfq(args.input) as src_store:
            inherited = (src_store.header.extra or {}).get(rp.HEADER_KEY)
    sampling = rp.profile_for_new_checkpoint(args.input if Path(str(args.input)).is_dir() else None,
                                             {"model_type": cfg.get("model_type") or cfg.get("family"), "_name_or_path": Path(str(args.input)).name},
                                             assets=assets, explicit=args.runtime_profile, inherited=inherited)
    if sampling is not None:
        extra[rp.HEADER_KEY] = sampling
    shard_bytes = int(args.shard_size_gb * (1 << 30)) if args.shard_size_gb else None
    if args.split_max_size:
        from .quantize.recipe import parse_size
        shard_bytes = parse_size(args.split_max_size)
    if base_records is not None:
        q = {**base_records, **q}
        extra["quantization"]["base_mfq"] = Path(args.base_mfq).name
    paths = save_checkpoint(out, cfg, q, assets, extra=extra, shard_bytes=shard_bytes, shard_tensors=args.split_max_tensors or None)
    size = sum(Path(p).stat().st_size for p in paths)
    weights = sum(int(t.size) for t in tensors.values())
    if store is not None:
        store.finish()
    print(json.dumps({"output": str(paths[0]), "shards": len(paths), "bytes": size, "weights": weights,
                      "bits_per_weight": round(8 * size / weights, 3), "resumed_tensors": len(store.reused) if store else 0}))
    return 0


def _alphaq_widths(tensors, target_bpw: float) -> dict[str, int]:
    """NINT width per 2-D weight from the AlphaQ allocation (heavier-tailed spectra get more bits) under the bit budget."""
    from .calibration import alphaq
    from .quantize import presets
    stats, sizes = {}, {}
    for name, t in tensors.items():
        if t.ndim == 2 and presets.quantizable(name, t.shape):
            stats[name] = alphaq.weight_statistics(t)
            sizes[name] = int(t.size)
    if not stats:
        return {}
    cands = {f"nint{b}": b + 0.3 for b in range(2, 9)}  # code bits + group parameters
    choice = alphaq.allocate(alphaq.importance(stats), sizes, cands, target_bpw * sum(sizes.values()))
    return {name: int(fam[4:]) for name, fam in choice.items()}


def _calibration_tokenizer(spec: str):
    """``byte`` = the byte-level tokenizer; else a ``tokenizer.json`` file or a directory that holds one (its
    ``tokenizer_config.json``, when present, supplies the chat template)."""
    from .server.tokenizer import ByteTokenizer, HfTokenizer
    if spec in ("", "byte"):
        return ByteTokenizer()
    p = Path(spec)
    root = p if p.is_dir() else p.parent
    blob = (root / "tokenizer.json" if p.is_dir() else p).read_bytes()
    template = eos = None
    if (root / "tokenizer_config.json").exists():
        tc = json.loads((root / "tokenizer_config.json").read_text())
        template, eos = tc.get("chat_template"), tc.get("eos_token") if isinstance(tc.get("eos_token"), str) else None
    return HfTokenizer(blob, chat_template=template, eos_token=eos)


def _cmd_calibrate_corpus(args) -> int:
    from .calibration import dataset
    tok = _calibration_tokenizer(args.tokenizer)
    if args.calibrate_cmd == "data":
        sources, files = {}, []
        for item in args.source:
            domain, _, path = item.rpartition("=")
            path = Path(path)
            files.append(path)
            sources.setdefault(domain or path.stem, []).extend(dataset.read_records(path))
        weights = {k: float(v) for k, v in (w.split("=") for w in args.domain_weight)} if args.domain_weight else None
        corpus = dataset.build_text_corpus(tok, args.output, sources, train_tokens=args.train_tokens,
                                           validation_tokens=args.validation_tokens, sequence_length=args.sequence_length,
                                           seed=args.seed, render_mode=args.render_mode, domain_weights=weights, source_files=files)
        event = "calibration_corpus_ready"
    else:
        rows, files = [], []
        for f in args.source_file:
            files.append(Path(f))
            rows.extend(dataset.read_records(f))
        corpus = dataset.build_trace_corpus(tok, args.output, rows, train_tokens=args.train_tokens,
                                            validation_tokens=args.validation_tokens, sequence_length=args.sequence_length,
                                            seed=args.seed, expected_generator_model=args.expected_generator_model or None,
                                            source_files=files)
        event = "trace_calibration_corpus_ready"
    print(json.dumps({"event": event, "path": str(corpus.root), "train_tokens": corpus.token_count("train"),
                      "validation_tokens": corpus.token_count("validation"), "windows": corpus.chunks,
                      "token_sha256": corpus.manifest["token_sha256"]}))
    return 0


def _cmd_calibrate(args) -> int:
    if args.calibrate_cmd in ("data", "trace-data"):
        return _cmd_calibrate_corpus(args)
    cfg, tensors, _assets = _load_source(args)
    if args.calibrate_cmd == "collect":
        from .calibration.dataset import load_corpus
        from .calibration.statistics import collect_statistics
        from .models.moe_lm import MoeConfig
        fields = MoeConfig.__dataclass_fields__
        mcfg = MoeConfig(**{k: v for k, v in cfg.items() if k in fields})
        stats = collect_statistics(mcfg, tensors, load_corpus(args.corpus), args.output, device=args.device,
                                   train_input_tokens=args.train_input_tokens, validation_input_tokens=args.validation_input_tokens,
                                   train_fisher_tokens=args.train_fisher_tokens, validation_fisher_tokens=args.validation_fisher_tokens,
                                   window=args.input_window or None, seed=args.seed)
        if args.imatrix_output:  # the input statistics in the form `mfq quantize --imatrix` reads
            np.savez(Path(args.imatrix_output), **stats.as_imatrix("train"))
        print(json.dumps({"event": "calibration_statistics_ready", "output": args.output, "tensors": len(stats.entries),
                          "mean_scored_loss": stats.metadata.get("mean_scored_loss")}))
        return 0
    if args.calibrate_cmd == "alphaq":
        from .calibration import alphaq
        from .quantize import presets
        stats, sizes = {}, {}
        for name, t in tensors.items():
            if not presets.quantizable(name, t.shape):
                continue
            if t.ndim == 3:
                for e in range(t.shape[0]):
                    stats[f"{name}#{e}"] = alphaq.weight_statistics(t[e])
                    sizes[f"{name}#{e}"] = int(t[e].size)
            else:
                stats[name] = alphaq.weight_statistics(t)
                sizes[name] = int(t.size)
        imp = alphaq.importance(stats)
        cands = {k: float(v) for k, v in (item.split(":") for item in args.candidates.split(","))}
        choice = alphaq.allocate(imp, sizes, cands, args.target_bpw * sum(sizes.values()))
        doc = {"format": "mfq.alphaq-allocation.v1", "target_bpw": args.target_bpw, "candidates": cands,
               "tensors": {k: {"alpha": stats[k].alpha, "variance": stats[k].variance, "importance": imp[k], "family": choice[k]}
                           for k in stats}}
        Path(args.output).write_text(json.dumps(doc, indent=1))
        used = sum(sizes[k] * cands[c] for k, c in choice.items()) / max(1, sum(sizes.values()))
        print(json.dumps({"output": args.output, "tensors": len(stats), "bits_per_weight": round(used, 3)}))
        return 0
    if args.calibrate_cmd == "inint":
        from .calibration import inint
        from .calibration.imatrix import load as load_imatrix
        doc = inint.select_rows(tensors, args.target_bpw, imatrix=load_imatrix(args.imatrix) if args.imatrix else None,
                                low=args.low, high=args.high, device=args.device)
        Path(args.output).write_text(json.dumps(doc))
        print(json.dumps({"output": args.output, "tensors": len(doc["tensors"]), **doc["report"]}))
        return 0
    if args.calibrate_cmd in ("candidates", "allocate", "natscale"):
        from .calibration import natscale
        from .calibration.imatrix import load as load_imatrix
        im = load_imatrix(args.imatrix) if args.imatrix else None
        layers = None
        if getattr(args, "layers", ""):
            layers = set()
            for part in args.layers.split(","):
                lo, _, hi = part.partition("-")
                layers.update(range(int(lo), int(hi or lo) + 1))
        if getattr(args, "candidates_file", None):
            cands = json.loads(Path(args.candidates_file).read_text())
        else:
            cands = natscale.expert_candidates(tensors, [f.strip().upper() for f in args.families.split(",") if f.strip()], imatrix=im,
                                               layers=layers)
        if args.calibrate_cmd == "candidates":
            Path(args.output).write_text(json.dumps(cands))
            print(json.dumps({"output": args.output, "banks": len(cands["tensors"]), "families": cands["families"]}))
            return 0
        if args.calibrate_cmd == "allocate" and args.method == "milp":
            # the exact joint solver over the same candidates; every expert weighs the same without an importance file
            from .calibration.ew_solver import solve
            total = sum(ex["weights"] for t in cands["tensors"] for ex in t["experts"])
            from .calibration.ew_solver import IMPORTANCE_FORMAT
            scheme, report = solve({"format": IMPORTANCE_FORMAT, "mode": "score", "entries": []}, cands,
                                   args.target_bpw * total)
        else:
            sens = args.sensitivity or ("imatrix-energy" if im is not None else "uniform")
            scheme, report = natscale.allocate(cands, args.target_bpw, imatrix=im, tensors=tensors, tau=args.tau, sensitivity=sens)
        Path(args.output).write_text(json.dumps(scheme, indent=1))
        if args.report:
            Path(args.report).write_text(json.dumps(report, indent=1))
        print(json.dumps({"output": args.output, **{k: v for k, v in report.items() if not isinstance(v, (dict, list))}}))
        return 0
    # imatrix: run the fp32 reference model with recording linears
    import torch
    from .calibration.imatrix import ImatrixCollector
    from .models.moe_lm import MoeConfig, MoeLM
    fields = MoeConfig.__dataclass_fields__
    mcfg = MoeConfig(**{k: v for k, v in cfg.items() if k in fields})
    col = ImatrixCollector()
    model = MoeLM(mcfg, {k: torch.from_numpy(np.asarray(v, dtype=np.float32)) for k, v in tensors.items()}, observer=col.observe,
                  reap_observer=col.observe_reap)
    g = torch.Generator().manual_seed(args.seed)
    tokens = 0
    if getattr(args, "corpus", ""):
        # windows of a calibration corpus (`mfq calibrate data` / `trace-data`) instead of random ids
        from .calibration.dataset import load_corpus
        for toks, _mask in load_corpus(args.corpus).iter_chunks("train", max_tokens=args.chunks * args.ctx):
            ids = torch.from_numpy(np.ascontiguousarray(toks[: args.ctx])).long()
            if int(ids.max()) >= mcfg.vocab_size:
                raise SystemExit(f"the corpus holds token id {int(ids.max())}, the model's vocabulary ends at {mcfg.vocab_size - 1}")
            model.reset()
            model.forward(ids)
            tokens += int(ids.numel())
    else:
        for _ in range(args.chunks):
            model.reset()
            model.forward(torch.randint(0, mcfg.vocab_size, (args.ctx,), generator=g))
            tokens += args.ctx
    col.save(args.output)
    print(json.dumps({"output": args.output, "layers": len(col.sum_in), "tokens": tokens}))
    return 0


def _cmd_solve_ew(args) -> int:
    from .calibration.ew_solver import solve_files
    print(json.dumps(solve_files(args.importance, args.candidates, args.budget, args.output_scheme, args.report)))
    return 0


def _cmd_inspect(args) -> int:
    from . import formats as F
    with F.open_mfq(args.model) as store:
        rows = [{"name": n, "dtype": store.dtype(n), "bytes": r.nbytes} for n, r in store.records.items()]
        info = {"arch": store.header.model_arch, "version": store.header.version, "extra": store.header.extra,
                "tensors": len(rows), "bytes": sum(r["bytes"] for r in rows)}
        graph = store.assets().get("model_graph.json")
        if graph:
            from .formats.model_graph import parse_graph
            g = parse_graph(graph)
            info["graph"] = {"backbone": g.backbone, "text_layers": g.text_layers, "predictor_layers": g.predictor_layers,
                             "capabilities": list(g.capabilities)}
    by = {}
    for r in rows:
        by[r["dtype"]] = by.get(r["dtype"], 0) + r["bytes"]
    info["bytes_by_dtype"] = by
    if args.tensors:
        info["records"] = rows
    print(json.dumps(info, indent=1))
    return 0


def _cmd_eval(args) -> int:
    """KLD / top-1 of a quantized checkpoint against a baseline checkpoint on random or given token windows."""
    import torch
    from . import formats as F
    from .evaluation.kld import compare_logits
    from .models.moe_lm import MoeConfig, MoeLM, dequantize_checkpoint

    def load(path):
        with F.open_mfq(path) as store:
            cfg = json.loads(store.assets()["model_config.json"])
            tensors = {n: store[n] for n in store if not n.startswith("__mfq_asset__/")}
        fields = MoeConfig.__dataclass_fields__
        return MoeConfig(**{k: v for k, v in cfg.items() if k in fields}), dequantize_checkpoint(tensors)

    if str(args.base).endswith("_logit3_") or Path(args.base).suffix in (".logit3", ".ref"):
        # the baseline is a reference-logits file (written by `mfq wt2-reference` or by the reference's own tool)
        from .evaluation.reference_logits import score_against_reference
        cfg, test = load(args.model)
        lm = MoeLM(cfg, test)
        rep = score_against_reference(args.base, lambda ids: lm.forward(torch.as_tensor(ids.astype("int64"))).float().numpy())
        print(" ".join(f"{k}={v:.6g}" if isinstance(v, float) else f"{k}={v}" for k, v in rep.items()))
        return 0
    cfg, base = load(args.base)
    _, test = load(args.model)
    g = torch.Generator().manual_seed(args.seed)
    reports = []
    rounding = None
    if getattr(args, "activation_q8", False):
        from .formats.nint8one import fake_quantize_nint8_one
        rounding = fake_quantize_nint8_one  # the tested model sees Q8_1-rounded projection inputs, the baseline does not
    for _ in range(args.chunks):
        ids = torch.randint(0, cfg.vocab_size, (args.ctx,), generator=g)
        lb, lt = MoeLM(cfg, base).forward(ids), MoeLM(cfg, test, input_transform=rounding).forward(ids)
        half = args.ctx // 2  # score the second half of each window, like the reference protocol
        reports.append(compare_logits(lb[half:], lt[half:]))
    n = len(reports)
    print(f"kld={sum(r.kld for r in reports) / n:.6g} mean_kld_q_ref={sum(r.reverse_kld for r in reports) / n:.6g} "
          f"same_top={100 * sum(r.top1_agreement for r in reports) / n:.2f}% chunks={n}")
    return 0


def _cmd_optimize_layout(args) -> int:
    """Rewrite a checkpoint into the layout the runtime executes: projections and routed experts as E4M3 with 128x128
    fp32 multipliers (what the loader would otherwise produce from NINT / NVQ at every start), 4-bit tensors kept as
    they are with ``--keep-4bit`` (for ``serve --native-4bit``).  Norms, routers and embeddings stay bf16."""
    import numpy as np
    from . import formats as F
    from .checkpoint import quantize_tensors, save_checkpoint
    from .ops import w4 as w4ops
    out = Path(args.output)
    if out.exists() and not args.overwrite:
        raise SystemExit(f"{out} exists (use --overwrite)")
    kept, floats = {}, {}
    with F.open_mfq(args.input) as store:
        assets = store.assets()
        cfg = json.loads(assets.pop("model_config.json"))
        assets.pop("model_graph.json", None)  # rebuilt on save
        arch, extra = store.header.model_arch, dict(store.header.extra or {})
        for n in store:
            if n.startswith("__mfq_asset__/"):
                continue
            t = store[n]
            if args.keep_4bit and ".mlp.experts." not in n and w4ops.from_checkpoint_tensor(t) is not None:
                kept[n] = t
            else:
                floats[n] = np.asarray(F.dequantize(t), dtype=np.float32)
    q = quantize_tensors(floats, dense="fp8", expert_mix="FP8", device=args.device)
    q.update(kept)
    extra.pop("runtime_assets", None)
    extra["layout"] = {"kind": "native", "dense": "FP8-128SQ", "kept_4bit": sorted(kept)}
    save_checkpoint(out, cfg, q, assets, arch=arch, extra=extra)
    print(json.dumps({"output": str(out), "bytes": out.stat().st_size, "transcoded": len(floats), "kept_4bit": len(kept)}))
    return 0


def _cmd_wt2_reference(args) -> int:
    """Write the baseline's reference-logits file (``_logit3_`` format: per scored position the full distribution as
    uint16 log-probability codes) over token windows from a file of token ids or, without one, seeded random windows."""
    import numpy as np
    import torch
    from . import formats as F
    from .evaluation.reference_logits import write_reference
    from .models.moe_lm import MoeConfig, MoeLM, dequantize_checkpoint
    with F.open_mfq(args.model) as store:
        cfg_d = json.loads(store.assets()["model_config.json"])
        tensors = {n: store[n] for n in store if not n.startswith("__mfq_asset__/")}
    cfg = MoeConfig(**{k: v for k, v in cfg_d.items() if k in MoeConfig.__dataclass_fields__})
    lm = MoeLM(cfg, dequantize_checkpoint(tensors))
    if args.tokens:
        ids = np.fromfile(args.tokens, dtype="<i4")
        chunks = min(args.chunks, len(ids) // args.ctx)
        if chunks < 1:
            raise SystemExit(f"{args.tokens} holds fewer than {args.ctx} token ids")
        windows = ids[: chunks * args.ctx].reshape(chunks, args.ctx)
    else:
        g = torch.Generator().manual_seed(args.seed)
        windows = torch.randint(0, cfg.vocab_size, (args.chunks, args.ctx), generator=g).numpy().astype("<i4")
    nll = write_reference(args.output, windows, lambda w: lm.forward(torch.as_tensor(w.astype("int64"))).float().numpy())
    from .evaluation.reference_logits import scored_span
    scored = windows.shape[0] * scored_span(args.ctx)[1]
    print(json.dumps({"output": args.output, "chunks": int(windows.shape[0]), "ctx": args.ctx, "baseline_nll": nll,
                      "baseline_ppl": float(np.exp(nll / max(1, scored)))}))
    return 0


def _cmd_serve(args) -> int:
    import torch
    import uvicorn
    from .checkpoint import load_engine
    from .server import ModelService, create_app
    device = args.device if args.device not in (None, "auto") else ("cuda" if torch.cuda.is_available() else "cpu")
    ctx = None
    if args.tensor_parallel > 1 and args.layer_parallel > 1:
        raise SystemExit("--tensor-parallel and --layer-parallel are mutually exclusive")
    ranks = max(args.tensor_parallel, args.layer_parallel)
    if ranks > 1:
        from .server import tp_serve
        if not tp_serve.under_launcher():  # first invocation: become N ranks
            import subprocess
            return subprocess.call(tp_serve.launcher_argv(sys.argv[1:] if args._argv is None else args._argv, ranks))
        ctx = tp_serve.RankContext(device)
        device = ctx.device
    tp = {}
    if ctx is not None and args.layer_parallel > 1:  # contiguous layer ranges per rank, run one after the other
        split = [float(x) for x in args.layer_split.split(",")] if args.layer_split else None
        tp = dict(lp_rank=ctx.rank, lp_size=ctx.world, layer_split=split, collective=ctx.collective)
    elif ctx is not None:
        tp = dict(tp_rank=ctx.rank, tp_size=ctx.world, collective=ctx.collective)

    if ctx is not None and ctx.rank != 0:  # follower: mirror rank 0's engine calls until it shuts down
        from .parallel.spmd import follower_loop
        engine, _tok, _cfg = load_engine(args.model, device, max_batch=args.continuous_batching, max_seq_len=args.ctx_size,
                                         native_4bit=args.native_4bit, yarn_context_extension=args.yarn_context_extension, **tp)
        why = follower_loop(engine, ctx.log)
        print(f"rank={ctx.rank} follower_exit={why}", file=sys.stderr)
        ctx.finish()
        return 0 if why == "shutdown" else 1
    import logging
    logging.basicConfig(level=getattr(logging, str(args.log_level).upper(), logging.INFO))
    service = ModelService(max_instances=args.max_runtime_instances, max_queue=args.max_queue, queue_timeout=args.queue_timeout,
                           idle_timeout=args.runtime_idle_timeout or None)
    if args.worker_process and ctx is None:
        return _serve_with_worker(args, service, device)

    policies = None
    if args.data_dir:
        from .server.policies import PolicyStore
        policies = PolicyStore(Path(args.data_dir) / "policies.json")

    def loader(name_or_path):
        path = name_or_path if Path(name_or_path).exists() else args.model
        pol = policies.get(args.model_name or Path(name_or_path).stem) if policies is not None else {}
        ctx_size = int(pol.get("context", {}).get("max_context_tokens") or args.ctx_size)
        kv_gb = float(pol.get("memory", {}).get("kv_budget_gb") or args.kv_budget_gb)
        cache_gb = float(pol.get("memory", {}).get("moe_gpu_cache_gb") or args.moe_gpu_cache_gb)
        if not Path(name_or_path).exists() and args.model_dir:  # a model name: look it up in the model directory
            for cand in (Path(args.model_dir) / name_or_path, Path(args.model_dir) / f"{name_or_path}.mfq"):
                if cand.exists():
                    path = str(cand)
                    break
        slots = args.moe_gpu_cache_slots
        if slots is None and cache_gb:
            slots = _expert_slots_for(path, cache_gb)
        engine, tok, _cfg = load_engine(path, device, max_batch=args.continuous_batching, max_seq_len=ctx_size, **tp,
                                        native_4bit=args.native_4bit, expert_slots=slots,
                                        expert_graphs=getattr(args, "moe_cache_graphs", False),
                                        kv_budget_bytes=int(kv_gb * (1 << 30)) if kv_gb else None,
                                        yarn_context_extension=args.yarn_context_extension,
                                        mtp_draft_tokens=args.mtp_draft_tokens, mtp_adaptive=args.mtp_adaptive,
                                        mtp_dynamic_depth=args.mtp_dynamic_depth)
        if args.prefill_chunk_size not in (None, "auto"):
            engine.prefill_chunk = max(16, int(args.prefill_chunk_size))
        if ctx is not None:
            # sharded serving: every rank must run the same kernels for a request, so the per-rank caches that let
            # rank 0 skip part of a prefill (session snapshots, prefix blocks) stay off
            return engine, tok
        if args.session_cache_gb > 0:
            from .engine.session_cache import SessionSnapshotCache
            engine.session_cache = SessionSnapshotCache(int(args.session_cache_gb * (1 << 30)))
        if args.prefix_cache_dir and not args.no_prefix_cache:
            from . import native
            from .quantize.recipe import parse_size
            ram = parse_size(args.prefix_cache_hot_size) if args.prefix_cache_hot_size else int(args.prefix_cache_ram_gb * (1 << 30))
            disk = parse_size(args.prefix_cache_disk_size) if args.prefix_cache_disk_size else int(args.prefix_cache_disk_gb * (1 << 30))
            engine.prefix_cache = native.PrefixCache(args.prefix_cache_dir, ram_budget=ram, disk_budget=disk,
                                                     block_tokens=args.prefix_cache_block_tokens)
            engine.prefix_salt = f"{Path(path).name}:{Path(path).stat().st_size}"
        return engine, tok

    service.loader = loader if ctx is None else None  # ranks load together at start; no loading on demand under TP
    engine, tok = loader(args.model)
    profile_path = None
    if args.moe_cache_profile:
        from .engine import moe_cache_profile as mcp
        profile_path = args.moe_cache_profile + (f".rank{ctx.rank}" if ctx is not None else "")
        warmed = mcp.apply(engine.model, mcp.load(profile_path))
        print(f"moe_cache_profile path={profile_path} warmed_experts={warmed}", file=sys.stderr)
    served_engine = engine
    if ctx is not None:
        from .parallel.spmd import LeaderBackend
        engine = LeaderBackend(engine, ctx.log)
    service.add_model(args.model_name or Path(args.model).stem, engine, tok)
    key = os.environ.get(args.api_key_env) if args.api_key_env else None
    if args.api_keys_file:
        from .server.auth import KeyStore
        store = KeyStore(args.api_keys_file)
        if key:
            store.add(key, ("admin",), name="startup key")
        key = store
    cluster = None
    if args.cluster_peer:
        from .server.cluster import ClusterBackend
        cluster = ClusterBackend(args.cluster_peer)
    sessions = None
    if args.db or args.data_dir:
        from .server.sessions import SessionStore
        db = Path(args.db) if args.db else Path(args.data_dir) / "mfq-server.sqlite3"
        db.parent.mkdir(parents=True, exist_ok=True)
        sessions = SessionStore(db)
    app = create_app(service, api_key=key, cluster=cluster, sessions=sessions, policies=policies)
    try:
        if args.anthropic_port and args.anthropic_port != args.port:
            from .server.listen import Listeners
            Listeners(app, args.host, [args.port, args.anthropic_port], access_log=args.access_log).start().wait()
        else:
            uvicorn.run(app, host=args.host, port=args.port, access_log=args.access_log)
    finally:
        if profile_path:
            mcp.save(profile_path, mcp.collect(served_engine.model, args.model_name or Path(args.model).stem))
        if ctx is not None:  # the server is down: let the other ranks go
            service.shutdown()
            engine.shutdown_followers()
            ctx.finish()
    return 0


def _expert_slots_for(path, gigabytes: float) -> int | None:
    """``--moe-gpu-cache-gb``: how many routed experts per layer fit in that much HBM (FP8 gate_up + down + multipliers)."""
    from . import formats as F
    if Path(path).is_dir():
        return None
    with F.open_mfq(path) as store:
        cfg = json.loads(store.assets()["model_config.json"])
    h, i, layers = int(cfg.get("hidden_size", 0)), int(cfg.get("moe_intermediate", 0) or 0), int(cfg.get("num_layers", 1))
    if not h or not i or not cfg.get("num_experts"):
        return None
    per_expert = 3 * h * i * (1 + 4 / (128 * 128))
    slots = int(gigabytes * (1 << 30) / (layers * per_expert))
    return max(1, slots) if slots < int(cfg["num_experts"]) else None


def _serve_with_worker(args, service, device) -> int:
    """``mfq serve --worker-process``: the engine lives in a child ``mfq runtime``; this process keeps HTTP, the
    tokenizer and the watch over the child (a dead child fails its requests at once and is restarted on demand)."""
    import uvicorn
    from . import formats as F
    from .server import create_app
    from .server.tokenizer import tokenizer_from_assets
    with F.open_mfq(args.model) as store:
        assets = store.assets()
    vocab = int(json.loads(assets["model_config.json"]).get("vocab_size", 0))
    command = [sys.executable, "-m", "mfq_b200.cli", "runtime", "--model", args.model, "--device", device,
               "--continuous-batching", str(args.continuous_batching), "--ctx-size", str(args.ctx_size),
               "--max-queue", str(args.max_queue), "--queue-timeout", str(args.queue_timeout),
               *(["--native-4bit"] if args.native_4bit else []),
               *(["--yarn-context-extension", str(args.yarn_context_extension)] if args.yarn_context_extension else [])]
    service.add_worker_model(args.model_name or Path(args.model).stem, command, tokenizer_from_assets(assets, vocab),
                             capacity=args.continuous_batching, ready_timeout=args.runtime_startup_timeout,
                             stall_timeout=args.runtime_stall_timeout or None)
    key = os.environ.get(args.api_key_env) if args.api_key_env else None
    try:
        uvicorn.run(create_app(service, api_key=key), host=args.host, port=args.port, access_log=args.access_log)
    finally:
        service.shutdown()
    return 0


def _cmd_runtime(args) -> int:
    """One model behind the newline-delimited JSON protocol on stdin / stdout (what a benchmark harness or a parent
    process drives; reference: the ``mfq-runtime --transport stdio`` executable, cpp_runtime/main.cpp)."""
    import torch
    from .checkpoint import load_engine
    from .server import ModelService
    from .server.stdio import StdioTransport
    device = args.device or ("cuda" if torch.cuda.is_available() else "cpu")
    out = sys.stdout
    sys.stdout = sys.stderr  # anything printed while serving must not corrupt the frame stream
    service = ModelService(max_queue=args.max_queue, queue_timeout=args.queue_timeout)
    engine, tok, _cfg = load_engine(args.model, device, max_batch=args.continuous_batching, max_seq_len=args.ctx_size,
                                    native_4bit=args.native_4bit, yarn_context_extension=args.yarn_context_extension)
    service.add_model(args.model_name or Path(args.model).stem, engine, tok)
    try:
        StdioTransport(service, sys.stdin, out).serve()
    finally:
        service.shutdown()
        sys.stdout = out
    return 0


def _cmd_profile(args) -> int:
    """Per-op time split of one prefill and a few eager decode steps (named scopes, CUDA events on a GPU)."""
    import torch
    from .checkpoint import load_engine
    from .utils.profiler import PROFILER, profile_engine
    device = args.device or ("cuda" if torch.cuda.is_available() else "cpu")
    engine, _tok, cfg = load_engine(args.model, device, max_batch=1, max_seq_len=args.prompt_tokens + args.decode_tokens + 8)
    vocab = int(cfg.vocab_size)
    ids = torch.tensor([3 + (i * 7919) % (vocab - 8) for i in range(args.prompt_tokens)], dtype=torch.int32)
    profile_engine(engine, ids, args.decode_tokens, args.filter)
    PROFILER.report(sys.stdout)
    return 0


def _cmd_bench_model(args) -> int:
    """Prompt-length x concurrency matrix through the stdio runtime; JSON (+ Markdown / HTML) report."""
    from .evaluation import model_bench as mb
    ints = lambda text: [int(x) for x in text.split(",") if x]
    if args.render:
        report = json.loads(Path(args.render).read_text())
    else:
        if not args.model and not args.runtime_command:
            raise SystemExit("--model (or --runtime-command) is required")
        command = args.runtime_command.split() if args.runtime_command else [
            sys.executable, "-m", "mfq_b200.cli", "runtime", "--model", args.model, "--continuous-batching",
            str(max(ints(args.concurrency))), "--ctx-size", str(max(ints(args.prompt_tokens)) + args.new_tokens + 16),
            *(["--device", args.device] if args.device else [])]
        report = mb.benchmark(command, ints(args.prompt_tokens), args.new_tokens, ints(args.concurrency), args.repeats,
                              args.warmup, mtp=args.mtp, label=args.label or (Path(args.model).stem if args.model else ""))
    problems = mb.validate_report(report)
    for line in problems:
        print(f"invalid report: {line}", file=sys.stderr)
    if args.output:
        Path(args.output).write_text(json.dumps(report, indent=1))
    if args.html:
        Path(args.html).write_text(mb.render_html(report))
    print(mb.render_markdown(report))
    return 1 if problems else 0


def _cmd_config(args) -> int:
    """The effective runtime configuration and the table of ``MFQ_*`` variables."""
    from .config import RuntimeConfig
    cfg = RuntimeConfig.from_env()
    rows = cfg.describe()
    if args.json:
        print(json.dumps(rows, indent=1))
        return 0
    for r in rows:
        mark = "" if r["value"] == r["default"] else "   (set)"
        print(f"{r['variable']:<22} = {r['value']!s:<10} default {r['default']!s:<8}{mark}\n    {r['what']}")
    return 0


def _cmd_bench(args) -> int:
    os.execv(sys.executable, [sys.executable, str(Path(__file__).resolve().parents[1] / "bench.py"), *args.rest])


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="mfq", description="Mixed-format quantization and serving on Blackwell GPUs")
    sub = ap.add_subparsers(dest="command", required=True)
    b = sub.add_parser("build", help="compile the sm_100a CUDA library")
    b.add_argument("--force", action="store_true")
    b.add_argument("--verbose", action="store_true")
    b.add_argument("--manifest", default="build/mfq-runtime.json")
    b.set_defaults(fn=_cmd_build)
    q = sub.add_parser("quantize", help="convert a Hugging Face directory / .mfq / synthetic model to a packed .mfq")
    q.add_argument("input")
    q.add_argument("output")
    q.add_argument("--bits", type=int, default=4)
    q.add_argument("--groupsize", type=int, default=0)
    q.add_argument("--sub-bits", type=int, default=0)
    q.add_argument("--format", choices=["nint2", "nint3", "nint4", "nint5", "nint6", "nint8", "nvq3", "mxfp4", "fp8", "bf16", "npq0-s", "npq0-l",
                                        "nvq1-l", "nvq1-l-s4", "nvq1-s", "nvq2j", "nvq2j-l", "nvq2j-xl", "nvq3j", "nvq3j-512", "nvq3j-l"],
                   help="family of every 2-D weight (and of routed experts without a mix): NINT widths, lattice / product codes, MX, FP8")
    q.add_argument("--preset", help="role-based mixed-width NINT preset: S2-S S2-M S3-S S3-M S3-L S4-S S4-M S5-S S5-M S6 S8")
    q.add_argument("--imatrix", help="importance matrix (.npz from `mfq calibrate imatrix`) for the NINT search")
    q.add_argument("--ew-scheme", "--scheme", dest="ew_scheme", help="mfq.calibration-scheme.v3 from `mfq solve-ew`")
    q.add_argument("--row-widths", help="per-neuron NINT widths (mfq.inint-rows.v1 from `mfq calibrate inint`)")
    q.add_argument("--random-expert-mix", default="", help="comma separated families per routed expert projection")
    q.add_argument("--random-expert-mix-seed", type=int, default=20260908)
    q.add_argument("--full-precision", action="store_true")
    q.add_argument("--device", "--backend", dest="device", default="cpu")
    q.add_argument("--seed", type=int, default=0)
    q.add_argument("--base-mfq", help="existing checkpoint to extend: its records are kept as they are and the source's multi-token-prediction head is added")
    q.add_argument("--recipe", help="per-tensor precisions from a GGUF file's tensor table (.gguf) or a JSON rule list")
    q.add_argument("--target-bpw", type=float, default=0.0, help="AlphaQ allocation of NINT widths over the 2-D weights under this budget")
    q.add_argument("--fp8-sq-bits", type=float, default=0.0,
                   help="with --format fp8: re-encode the E4M3 tensors with per-row scalar palettes (FP8-128SQ rows SQ1..SQ8) "
                        "averaging this many code bits per weight")
    q.add_argument("--runtime-profile", help="runtime.sampling.v1 JSON whose sampling defaults are embedded in the output "
                                             "(over the architecture registry, the source's generation config and its mfq-runtime.json)")
    q.add_argument("--mxfp4-sq-bits", type=float, default=0.0,
                   help="re-code every MXFP4 matrix (dense with --format mxfp4, expert pools of a mix) as MXFP4-SQ: rows of 1..4 "
                        "symbol bits over catalogue palettes, averaging this many stored bits per weight; still legal MXFP4 once decoded")
    q.add_argument("--split-max-size", help="limit of tensor payload per output shard, N[M|G]")
    q.add_argument("--split-max-tensors", type=int, default=0, help="limit of tensors per output shard")
    q.add_argument("--dry-run", action="store_true")
    q.add_argument("--resume", action="store_true", help="reuse the validated per-tensor blobs an interrupted run left in <output>.tmp/")
    q.add_argument("--resume-completed", action="store_true", help="exit at once when the output already exists and opens")
    q.add_argument("--keep-temp", action="store_true", help="keep <output>.tmp/ after a successful run")
    q.add_argument("--no-temp", action="store_true", help="do not park finished tensors on disk while quantizing")
    q.add_argument("--overwrite", action="store_true")
    q.add_argument("--verbose", action="store_true")
    q.add_argument("--shard-size-gb", type=float, default=0.0, help="write name-0000i-of-0000N.mfq shards of at most this size")
    q.set_defaults(fn=_cmd_quantize)
    c = sub.add_parser("calibrate", help="importance statistics for bit allocation")
    cs = c.add_subparsers(dest="calibrate_cmd", required=True)
    ca = cs.add_parser("alphaq", help="calibration-free spectral importance of every 2-D / expert weight + allocation")
    ca.add_argument("input")
    ca.add_argument("--target-bpw", type=float, default=4.0)
    ca.add_argument("--candidates", default="NINT2:2.6,NINT3:3.6,NINT4:4.5,NINT5:5.5,NINT6:6.5,NINT8:8.5")
    ca.add_argument("--output", required=True, help="JSON: per-tensor alpha / variance / importance / chosen family")
    ca.add_argument("--seed", type=int, default=0)
    ci = cs.add_parser("imatrix", help="input-channel importance of every linear layer on random or given token windows")
    ci.add_argument("input")
    ci.add_argument("--output", required=True)
    ci.add_argument("--chunks", type=int, default=4)
    ci.add_argument("--ctx", type=int, default=128)
    ci.add_argument("--corpus", default="", help="calibration corpus directory (`mfq calibrate data`); default: random token ids")
    ci.add_argument("--seed", type=int, default=0)
    cd = cs.add_parser("data", help="tokenize local text / JSONL records into a train + validation calibration corpus")
    cd.add_argument("--source", action="append", required=True, metavar="[DOMAIN=]FILE",
                    help="JSONL ({\"text\"} or {\"messages\"} per line) or plain text (paragraphs); repeatable")
    cd.add_argument("--domain-weight", action="append", default=[], metavar="DOMAIN=W", help="share of a domain in both splits (default equal)")
    cd.add_argument("--render-mode", choices=("auto", "plain"), default="auto", help="plain: never apply the chat template")
    ct = cs.add_parser("trace-data", help="tokenize model-generated JSONL traces; only generated positions are scored")
    ct.add_argument("--source-file", action="append", required=True)
    ct.add_argument("--expected-generator-model", default="", help="reject rows whose `model` differs")
    for p_ in (cd, ct):
        p_.add_argument("--tokenizer", default="byte", help="tokenizer.json, a directory holding one, or `byte`")
        p_.add_argument("--output", required=True, help="corpus directory to create")
        p_.add_argument("--train-tokens", type=int, default=1 << 20)
        p_.add_argument("--validation-tokens", type=int, default=1 << 17)
        p_.add_argument("--sequence-length", type=int, default=2048)
        p_.add_argument("--seed", type=int, default=0)
        p_.set_defaults(fn=_cmd_calibrate)
    cc = cs.add_parser("collect", help="activation second moments and row Fisher of every linear layer over a corpus")
    cc.add_argument("input")
    cc.add_argument("--corpus", required=True, help="directory written by `calibrate data` / `calibrate trace-data`")
    cc.add_argument("--output", required=True, help=".npz statistics file to create")
    cc.add_argument("--imatrix-output", default="", help="also write the input statistics as an importance matrix")
    cc.add_argument("--device", default="cpu")
    cc.add_argument("--input-window", type=int, default=0, help="truncate every window to this many tokens (0: whole windows)")
    cc.add_argument("--train-input-tokens", type=int, default=1 << 16)
    cc.add_argument("--validation-input-tokens", type=int, default=1 << 14)
    cc.add_argument("--train-fisher-tokens", type=int, default=1 << 14)
    cc.add_argument("--validation-fisher-tokens", type=int, default=1 << 12)
    cc.add_argument("--seed", type=int, default=0)
    cc.set_defaults(fn=_cmd_calibrate)
    def _candidate_args(p, target=True):
        p.add_argument("input")
        p.add_argument("--families", default="NINT2,NINT3,NINT4,NINT5,NINT6,NINT8", help="NINT families scored per expert matrix")
        p.add_argument("--imatrix", help="importance matrix with per-expert statistics (`mfq calibrate imatrix`)")
        p.add_argument("--layers", default="", help="comma-separated layers or ranges (default: all)")
        p.add_argument("--seed", type=int, default=0)
        p.add_argument("--output", required=True)
        if target:
            p.add_argument("--candidates-file", help="reuse a table written by `mfq calibrate candidates`")
            p.add_argument("--target-bpw", type=float, required=True, help="mean bits per routed-expert weight")
            p.add_argument("--tau", type=float, default=1.0, help="NatScale contrast in nats")
            p.add_argument("--sensitivity", choices=("uniform", "imatrix-energy", "reap"), default=None)
            p.add_argument("--report")
    cc = cs.add_parser("candidates", help="quantize every routed expert matrix under every family: error and size table")
    _candidate_args(cc, target=False)
    cl = cs.add_parser("allocate", help="score candidates and allocate a family per expert matrix under a budget")
    _candidate_args(cl)
    cl.add_argument("--method", choices=("natscale", "milp"), default="natscale")
    cn = cs.add_parser("natscale", help="NatScale allocation (contrast-normalised sensitivities, convex-hull budget solver)")
    _candidate_args(cn)
    cr = cs.add_parser("inint", help="per-neuron NINT widths: every row of every dense projection narrow or wide under a budget")
    cr.add_argument("input")
    cr.add_argument("--imatrix")
    cr.add_argument("--target-bpw", type=float, required=True)
    cr.add_argument("--low", type=int, default=4)
    cr.add_argument("--high", type=int, default=8)
    cr.add_argument("--device", default="cpu")
    cr.add_argument("--seed", type=int, default=0)
    cr.add_argument("--output", required=True)
    for p_ in (cc, cl, cn, cr):
        p_.set_defaults(fn=_cmd_calibrate)
    se = sub.add_parser("solve-ew", help="expert-wise joint budget solver (MILP) -> calibration scheme")
    se.add_argument("--importance", required=True)
    se.add_argument("--candidates", required=True)
    se.add_argument("--budget", required=True)
    se.add_argument("--output-scheme", required=True)
    se.add_argument("--report")
    se.set_defaults(fn=_cmd_solve_ew)
    ca.set_defaults(fn=_cmd_calibrate)
    ci.set_defaults(fn=_cmd_calibrate)

    dg = sub.add_parser("diagnose", help="self-checks: formats anywhere, kernels and the engine on a GPU box")
    dg.add_argument("--check", action="append", help="run only this check (repeatable); `mfq diagnose --list` prints the names")
    dg.add_argument("--list", action="store_true", help="print the names of all checks and exit")
    from . import diagnostics as _diag
    dg.set_defaults(fn=_diag.main)
    i = sub.add_parser("inspect", help="summarise an .mfq container")
    i.add_argument("model")
    i.add_argument("--tensors", action="store_true")
    i.set_defaults(fn=_cmd_inspect)
    e = sub.add_parser("eval", help="quality evaluation")
    es = e.add_subparsers(dest="what", required=True)
    kl = es.add_parser("kl", help="KLD / top-1 agreement against a baseline checkpoint")
    kl.add_argument("--model", required=True)
    kl.add_argument("--base", "--kl-base", dest="base", required=True)
    kl.add_argument("--chunks", "--kl-chunks", dest="chunks", type=int, default=4)
    kl.add_argument("--ctx", type=int, default=128)
    kl.add_argument("--seed", type=int, default=0)
    kl.add_argument("--activation-q8", action="store_true",
                    help="round the inputs of the tested model's projections to NINT8-1 (Q8_1) blocks, as an int8-activation runtime does")
    kl.set_defaults(fn=_cmd_eval)
    ol = sub.add_parser("optimize-layout", aliases=["optimize"], help="rewrite a checkpoint into the runtime's native execution layout")
    ol.add_argument("--input", required=True)
    ol.add_argument("--output", required=True)
    ol.add_argument("--overwrite", action="store_true")
    ol.add_argument("--keep-4bit", action="store_true", help="leave NINT (<= 4 bits) / MXFP4 projections as they are")
    ol.add_argument("--device", default="cpu")
    ol.set_defaults(fn=_cmd_optimize_layout)
    wr = sub.add_parser("wt2-reference", help="write a baseline's reference-logits file (_logit3_) for `eval kl --base`")
    wr.add_argument("--model", required=True, help="baseline .mfq (usually the full-precision checkpoint)")
    wr.add_argument("--output", required=True)
    wr.add_argument("--tokens", help="little-endian int32 token ids (e.g. a tokenized WikiText-2 test split); default: random windows")
    wr.add_argument("--chunks", type=int, default=4)
    wr.add_argument("--ctx", type=int, default=128)
    wr.add_argument("--seed", type=int, default=0)
    wr.set_defaults(fn=_cmd_wt2_reference)
    s = sub.add_parser("serve", help="OpenAI/Anthropic-compatible server")
    s.add_argument("--model", required=True)
    s.add_argument("--model-name")
    s.add_argument("--host", default="127.0.0.1")
    s.add_argument("--port", type=int, default=8090)
    s.add_argument("--api-key-env")
    s.add_argument("--continuous-batching", "--max-requests-per-runtime", dest="continuous_batching", type=int, default=32)
    s.add_argument("--ctx-size", "--context-size", dest="ctx_size", type=int, default=8192)
    s.add_argument("--prefill-chunk-size", default="auto", help="auto, or the longest prompt span prefilled in one pass")
    s.add_argument("--max-runtime-instances", type=int, default=1)
    s.add_argument("--max-queue", "--max-queued-requests-per-runtime", dest="max_queue", type=int, default=256)
    s.add_argument("--queue-timeout", type=float, default=30.0)
    s.add_argument("--runtime-idle-timeout", type=float, default=0.0, help="unload a model idle for this many seconds (0: never)")
    s.add_argument("--model-dir", help="directory in which model names given to /api/v1/models/load are looked up")
    s.add_argument("--data-dir", help="directory of the server's own state (session database)")
    s.add_argument("--db", help="SQLite file of the session store (default: in memory, or <data-dir>/mfq-server.sqlite3)")
    s.add_argument("--moe-gpu-cache-gb", type=float, default=0.0, help="HBM for routed experts; the rest stay in pinned host memory")
    s.add_argument("--moe-cache-profile", help="JSON file of expert heat: warms the HBM expert arena at start, rewritten at shutdown")
    s.add_argument("--prefix-cache-disk-size", help="N[M|G]; overrides --prefix-cache-disk-gb")
    s.add_argument("--prefix-cache-hot-size", help="N[M|G]; overrides --prefix-cache-ram-gb")
    s.add_argument("--prefix-cache-block-tokens", type=int, default=256)
    s.add_argument("--no-prefix-cache", action="store_true")
    s.add_argument("--log-level", default="info")
    s.add_argument("--device", "--backend", dest="device")
    s.add_argument("--access-log", action="store_true")
    s.add_argument("--native-4bit", action="store_true",
                   help="run NINT (<= 4 code bits) / MXFP4 projections through the 4-bit in-pipeline-decode GEMM instead of FP8")
    s.add_argument("--moe-gpu-cache-slots", type=int, default=None,
                   help="keep routed experts in pinned host memory behind an HBM arena of this many slots per layer")
    s.add_argument("--moe-cache-graphs", action="store_true",
                   help="with an expert cache: decode inside CUDA graphs with the resident experts and replay a step "
                        "after uploading what it missed (without it such a model decodes eagerly, in waves)")
    s.add_argument("--mtp-draft-tokens", type=int, default=0,
                   help="draft this many tokens per cycle with the checkpoint's multi-token-prediction head (0: off)")
    s.add_argument("--mtp-dynamic-depth", action="store_true",
                   help="choose the number of drafts (1 .. --mtp-draft-tokens) per cycle from measured tokens per millisecond")
    s.add_argument("--mtp-adaptive", action="store_true",
                   help="measure cycles against plain decoding and park them while they lose (the head stays primed)")
    s.add_argument("--runtime-startup-timeout", type=float, default=600.0, help="seconds a worker process may take to announce itself")
    s.add_argument("--runtime-stall-timeout", type=float, default=300.0,
                   help="a worker with requests in flight that sends nothing for this long is killed as hung (0: never)")
    s.add_argument("--worker-process", action="store_true",
                   help="run the engine in a child process that is watched and restarted on demand (the server survives a dead engine)")
    s.add_argument("--tensor-parallel", type=int, default=1,
                   help="ranks (one process per GPU) that share every layer: attention heads, FFN columns and experts are sharded")
    s.add_argument("--layer-parallel", type=int, default=1,
                   help="ranks that each hold a contiguous range of layers (weights and KV) and run one after the other")
    s.add_argument("--layer-split", help="comma separated weights of the layer ranges, e.g. 3,1")
    s.add_argument("--expert-parallel", action="store_true",
                   help="accepted for compatibility: the ranks of --tensor-parallel always split the routed experts among themselves too")
    s.add_argument("--yarn-context-extension", type=float, default=None,
                   help="run on this multiple (> 1) of the trained context with YaRN-scaled rotary frequencies")
    s.add_argument("--anthropic-port", type=int, default=0,
                   help="second listener for Anthropic-style clients (the reference uses 8091); 0: one port serves both")
    s.add_argument("--api-keys-file", default=None,
                   help="JSON store of API keys with scopes (inference / read / admin); keys are kept as SHA-256 digests")
    s.add_argument("--kv-budget-gb", type=float, default=0.0,
                   help="cap of the paged KV pool (default on a GPU: 90%% of the memory free after loading the weights)")
    s.add_argument("--cluster-peer", action="append", default=[],
                   help="base URL of another server of this kind; models it serves are routed there (repeatable)")
    s.add_argument("--session-cache-gb", type=float, default=8.0,
                   help="host memory for per-conversation KV (+ recurrent state) snapshots, keyed by the request's session_id (0: off)")
    s.add_argument("--prefix-cache-dir", default=None, help="directory of the content-addressed KV prefix cache (256-token blocks)")
    s.add_argument("--prefix-cache-ram-gb", type=float, default=4.0)
    s.add_argument("--prefix-cache-disk-gb", type=float, default=64.0)
    s.set_defaults(fn=_cmd_serve)
    bm = sub.add_parser("bench-model", help="prefill / decode / TTFT over a prompt-length x concurrency matrix (stdio runtime)")
    bm.add_argument("--model")
    bm.add_argument("--runtime-command", help="another runtime that speaks the stdio frames (instead of --model)")
    bm.add_argument("--prompt-tokens", default="128,1024")
    bm.add_argument("--new-tokens", type=int, default=64)
    bm.add_argument("--concurrency", default="1,8")
    bm.add_argument("--repeats", type=int, default=3)
    bm.add_argument("--warmup", type=int, default=1)
    bm.add_argument("--mtp", action="store_true")
    bm.add_argument("--device")
    bm.add_argument("--label", default="")
    bm.add_argument("--output", help="write the JSON report here")
    bm.add_argument("--html", help="write a self-contained HTML report here")
    bm.add_argument("--render", help="render an existing JSON report instead of running")
    bm.set_defaults(fn=_cmd_bench_model)
    cf = sub.add_parser("config", help="effective runtime configuration and the MFQ_* environment variables")
    cf.add_argument("--json", action="store_true")
    cf.set_defaults(fn=_cmd_config)
    pf = sub.add_parser("profile", help="per-op time split of a prefill and a few eager decode steps")
    pf.add_argument("--model", required=True)
    pf.add_argument("--prompt-tokens", type=int, default=128)
    pf.add_argument("--decode-tokens", type=int, default=8)
    pf.add_argument("--filter", default="", help="comma separated name pieces to keep (e.g. attn,ffn.down)")
    pf.add_argument("--device")
    pf.set_defaults(fn=_cmd_profile)
    rt = sub.add_parser("runtime", help="serve one model over newline-delimited JSON frames on stdin / stdout")
    rt.add_argument("--model", required=True)
    rt.add_argument("--model-name")
    rt.add_argument("--transport", choices=["stdio"], default="stdio")
    rt.add_argument("--continuous-batching", type=int, default=32)
    rt.add_argument("--ctx-size", type=int, default=8192)
    rt.add_argument("--max-queue", type=int, default=256)
    rt.add_argument("--queue-timeout", type=float, default=30.0)
    rt.add_argument("--native-4bit", action="store_true")
    rt.add_argument("--yarn-context-extension", type=float, default=None)
    rt.add_argument("--device")
    rt.set_defaults(fn=_cmd_runtime)
    be = sub.add_parser("bench", help="run the flagship benchmark (arguments are passed through to bench.py)")
    be.add_argument("rest", nargs=argparse.REMAINDER)
    be.set_defaults(fn=_cmd_bench)
    return ap


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
    args._argv = None if argv is None else list(argv)  # what a re-launch under the rank launcher repeats
    return int(args.fn(args) or 0)


if __name__ == "__main__":
    sys.exit(main())
