"""Checkpoint assembly and loading: Hugging Face directory / synthetic model -> ``.mfq`` -> engine.

``model_config.json`` travels as the runtime asset ``__mfq_asset__/model_config.json`` (the reference embeds its
runtime assets the same way, ``mfq/formats/assets.py:22-37``), tokenizer files under ``__mfq_asset__/hf/...``.
"""

from __future__ import annotations

import json
import struct
from pathlib import Path

import numpy as np
import torch

from . import formats as F
from .architectures import config_from_hf, to_canonical
from .formats.container import ASSET_PREFIX

_ST_DTYPES = {"F32": np.float32, "F16": np.float16, "BF16": np.uint16, "I64": np.int64, "I32": np.int32, "U8": np.uint8,
              "F8_E4M3": np.uint8}


def read_safetensors(path) -> dict[str, np.ndarray]:
    """Minimal safetensors reader (8-byte header length, JSON header, raw little-endian data); float32 output."""
    out = {}
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
        base = 8 + n
        for name, meta in header.items():
            if name == "__metadata__":
                continue
            a, b = meta["data_offsets"]
            f.seek(base + a)
            raw = np.frombuffer(f.read(b - a), dtype=_ST_DTYPES[meta["dtype"]]).reshape(meta["shape"])
            if meta["dtype"] == "BF16":
                raw = F.from_bf16(raw)
            elif meta["dtype"] == "F8_E4M3":
                from .formats.mx import e4m3_to_float
                raw = e4m3_to_float(raw)
            out[name] = np.asarray(raw, dtype=np.float32) if raw.dtype.kind == "f" else raw
    return out


def read_hf_directory(path) -> tuple[dict, dict[str, np.ndarray], dict[str, bytes]]:
    """(model config kwargs, canonical float32 tensors, tokenizer assets) of a Hugging Face checkpoint directory."""
    p = Path(path)
    hf_cfg = json.loads((p / "config.json").read_text())
    tensors: dict[str, np.ndarray] = {}
    for shard in sorted(p.glob("*.safetensors")):
        tensors.update(read_safetensors(shard))
    tensors = fold_source_quantization(tensors, hf_cfg)
    assets = {}
    for fname in ("tokenizer.json", "tokenizer_config.json", "generation_config.json", "chat_template.jinja"):
        if (p / fname).exists():
            assets[f"hf/{fname}"] = (p / fname).read_bytes()
    return config_from_hf(hf_cfg), to_canonical(tensors, hf_cfg), assets


def fold_source_quantization(tensors: dict[str, np.ndarray], hf_cfg: dict | None = None) -> dict[str, np.ndarray]:
    """Sources that ship already-quantized weights, folded to plain float32 matrices under their plain names:

    * block-scaled FP8 (``<w>`` in E4M3 with ``<w>_scale_inv`` of shape ``[ceil(out / b0), ceil(in / b1)]``; the block
      comes from ``quantization_config.weight_block_size``, default 128 x 128): ``w * scale_inv`` per block;
    * tensor- or channel-scaled FP8 (``<w>`` with ``<w>_scale`` holding one value, or one per output row);
      ``input_scale`` / ``activation_scale`` companions (static activation ranges) are dropped;
    * MXFP4 in the ``<name>_blocks`` / ``<name>_scales`` layout (``[..., groups, 16]`` bytes of two E2M1 nibbles, low
      first, and one E8M0 exponent per 32 values): ``<name>`` becomes ``[..., groups * 32]`` float32.

    Reference: the scaled-FP8 and MXFP4 source readers of ``mfq/formats/hf_source.py`` and ``mfq/convert/``."""
    from .formats.mx import E2M1_VALUES
    qc = (hf_cfg or {}).get("quantization_config") or {}
    block = tuple(qc.get("weight_block_size") or (128, 128))
    out = dict(tensors)
    for name in list(out):
        if name.endswith("_scale_inv") and name[: -len("_scale_inv")] in out:
            base = name[: -len("_scale_inv")]
            w, sc = np.asarray(out[base], dtype=np.float32), np.asarray(out.pop(name), dtype=np.float32)
            lead = w.shape[:-2]
            rows, cols = w.shape[-2:]
            if sc.shape != lead + (-(-rows // block[0]), -(-cols // block[1])):
                raise ValueError(f"{name}: scale grid {sc.shape} does not cover {w.shape} in {block[0]}x{block[1]} blocks")
            full = np.repeat(np.repeat(sc, block[0], axis=-2), block[1], axis=-1)[..., :rows, :cols]
            out[base] = w * full
        elif name.endswith(".weight_scale") and name[: -len("_scale")] in out:
            base = name[: -len("_scale")]
            w, sc = np.asarray(out[base], dtype=np.float32), np.asarray(out.pop(name), dtype=np.float32)
            if sc.size == 1:
                out[base] = w * sc.reshape(())
            elif sc.size == int(np.prod(w.shape[:-1])):
                out[base] = w * sc.reshape(w.shape[:-1] + (1,))
            else:
                raise ValueError(f"{name}: {sc.shape} is neither one scale nor one per output row of {w.shape}")
        elif name.endswith((".input_scale", ".activation_scale")):
            out.pop(name)
    for name in list(out):
        if name.endswith("_blocks") and name[: -len("_blocks")] + "_scales" in out:
            base = name[: -len("_blocks")]
            blocks, scales = np.asarray(out.pop(name)), np.asarray(out.pop(base + "_scales"))
            if blocks.dtype != np.uint8 or scales.dtype != np.uint8 or blocks.shape[-1] != 16 or blocks.shape[:-1] != scales.shape:
                raise ValueError(f"{name}: expected uint8 [..., groups, 16] with uint8 exponents [..., groups]")
            nib = np.stack([blocks & 15, blocks >> 4], -1).reshape(blocks.shape[:-1] + (32,))
            val = np.where(nib & 8, -E2M1_VALUES[nib & 7], E2M1_VALUES[nib & 7]).astype(np.float32)
            val = val * np.ldexp(np.float32(1.0), scales.astype(np.int32) - 127)[..., None]
            out[base] = val.reshape(blocks.shape[:-2] + (blocks.shape[-2] * 32,)).astype(np.float32)
    return out


def quantize_tensors(tensors: dict[str, np.ndarray], *, dense: str = "nint4", expert_mix: str = "", seed: int = 20260908,
                     device: str = "cpu", progress=None, widths: dict[str, int | None] | None = None,
                     imatrix: dict[str, np.ndarray] | None = None, scheme: dict | None = None, resume=None,
                     fp8_sq_bits: float = 0.0, row_widths: dict | None = None, mxfp4_sq_bits: float = 0.0) -> dict[str, object]:
    """Apply the quantization plan: routed experts by the seeded mix (or the dense rule), 2-D weights by ``dense``
    (nint2..8 / nvq3 / mxfp4 / fp8 / bf16), norms / router / embeddings-as-requested stay bf16.
    ``widths`` (a preset plan: tensor -> NINT width, None = keep) overrides ``dense`` per tensor; ``imatrix`` supplies
    per-input-channel importance to the NINT search; ``scheme`` (``mfq.calibration-scheme.v3``, expert-wise) fixes the
    family of every routed expert projection.  ``resume`` (a :class:`~mfq_b200.quantize.resume.ResumeStore`) parks
    every finished tensor and hands back the ones a previous, interrupted run finished for the same source and plan.
    ``fp8_sq_bits`` (1..8, 0 = off): dense FP8 tensors are re-encoded with per-row scalar palettes averaging that many
    code bits per weight (``quantize/fp8_sq.py``; the imatrix, if given, weights the palette fit).  ``row_widths``
    (``mfq.inint-rows.v1`` from ``mfq calibrate inint``): the listed tensors become NINT with a code width per output row.
    ``mxfp4_sq_bits`` (about 1.3 .. 4.25, 0 = off): every MXFP4 matrix -- dense, or a pool of routed experts -- is re-coded
    as MXFP4-SQ with per-row widths averaging that many stored bits per weight (``quantize/mxfp4_sq.py``)."""
    if resume is not None:
        if fp8_sq_bits or mxfp4_sq_bits or row_widths is not None:
            raise ValueError("--fp8-sq-bits / --row-widths cannot be combined with a resumable run yet")
        return _quantize_resumable(tensors, resume, dense=dense, expert_mix=expert_mix, seed=seed, device=device,
                                   progress=progress, widths=widths, imatrix=imatrix, scheme=scheme)
    from .quantize import balanced_expert_mix, parse_profiles, quantize_expertwise, quantize_matrix
    profiles = parse_profiles(expert_mix) if expert_mix else ()
    dense_profile = None if dense == "bf16" else parse_profiles({"fp8": "FP8", "mxfp4": "MXFP4", "nvq3": "NVQ3"}.get(dense, dense.upper()))[0]
    out: dict[str, object] = {}
    for name, t in tensors.items():
        if progress:
            progress(name)
        a = np.asarray(t, dtype=np.float32)
        keep = a.ndim < 2 or "norm" in name or "router" in name or name.endswith(".bias")
        profile = dense_profile
        if widths is not None and name in widths:
            profile = None if widths[name] is None else parse_profiles(f"NINT{widths[name]}")[0]
        if ".mlp.experts." in name and a.ndim == 3:
            fixed = [x for x in (scheme or {}).get("assignments", []) if x["tensor"] == name]
            if fixed:
                families = sorted({x["family"] for x in fixed})
                use = parse_profiles(",".join(families))
                assign = np.zeros(a.shape[0], dtype=np.int64)
                for x in fixed:
                    assign[int(x["expert_id"])] = families.index(x["family"])
                out[name] = quantize_expertwise(a, assign, tuple(use), device=device)
                continue
            use = profiles or ((profile,) if profile else ())
            if not use:
                out[name] = F.to_bf16(a)
                continue
            assign = balanced_expert_mix(name, a.shape[0], len(use), seed)
            out[name] = quantize_expertwise(a, assign, tuple(use), device=device)
        elif keep or profile is None or (profile.family in ("FP8", "MXFP4") and a.shape[-1] % 128):
            out[name] = F.to_bf16(a)
        elif row_widths is not None and name in row_widths.get("tensors", {}):
            from .calibration.imatrix import input_importance
            from .calibration.inint import row_bits
            from .quantize.nint import quantize_nint
            spec = parse_profiles(f"NINT{int(row_widths['low'])}")[0].nint
            imp = input_importance(imatrix, name) if imatrix is not None else None
            out[name] = quantize_nint(a, spec, row_q_bits=row_bits(row_widths, name), importance=imp, device=device)
        else:
            imp = None
            if imatrix is not None and profile.nint is not None:
                from .calibration.imatrix import input_importance
                imp = input_importance(imatrix, name)
            out[name] = quantize_matrix(a, profile, device=device, importance=imp) if imp is not None else quantize_matrix(a, profile, device=device)
            if fp8_sq_bits and profile.family == "FP8":
                from .calibration.imatrix import input_importance
                from .quantize.fp8_sq import quantize_fp8_sq
                weight = input_importance(imatrix, name) if imatrix is not None else None
                out[name] = quantize_fp8_sq(out[name], float(fp8_sq_bits), weight)
    if mxfp4_sq_bits:
        from .formats.mfe import MfePool, MfeTensor
        from .formats.mx import MXFP4_DTYPE, MxTensor
        from .quantize.mxfp4_sq import quantize_mxfp4_sq
        is_mx = lambda t: isinstance(t, MxTensor) and t.dtype == MXFP4_DTYPE
        for name, t in list(out.items()):
            if progress and (is_mx(t) or isinstance(t, MfeTensor)):
                progress(name + " [mxfp4-sq]")
            if is_mx(t):
                out[name] = quantize_mxfp4_sq(t, target_bits=float(mxfp4_sq_bits))
            elif isinstance(t, MfeTensor) and any(is_mx(p.tensor) for p in t.pools):
                out[name] = MfeTensor(t.shape, tuple(
                    MfePool(p.expert_ids, quantize_mxfp4_sq(p.tensor, target_bits=float(mxfp4_sq_bits)), p.runtime) if is_mx(p.tensor) else p
                    for p in t.pools))
    return out


def _quantize_resumable(tensors, store, *, dense, expert_mix, seed, device, progress, widths, imatrix, scheme):
    """One tensor at a time through :func:`quantize_tensors`, with the resume store in front of it."""
    import hashlib
    out: dict[str, object] = {}
    for name, t in tensors.items():
        a = np.asarray(t, dtype=np.float32)
        label = {"dense": dense, "mix": expert_mix, "seed": seed, "width": (widths or {}).get(name, "-") if widths is not None else "-",
                 "scheme": [x for x in (scheme or {}).get("assignments", []) if x["tensor"] == name]}
        if imatrix is not None:
            from .calibration.imatrix import input_importance
            imp = input_importance(imatrix, name)
            label["imatrix"] = None if imp is None else hashlib.sha256(np.ascontiguousarray(imp, dtype=np.float32).data).hexdigest()
        key = store.key(name, a, json.dumps(label, sort_keys=True))
        got = store.get(name, key)
        if got is None:
            got = quantize_tensors({name: a}, dense=dense, expert_mix=expert_mix, seed=seed, device=device, progress=progress,
                                   widths=widths, imatrix=imatrix, scheme=scheme)[name]
            store.put(name, key, got)
        out[name] = got
    return out


def save_checkpoint(path, config: dict, tensors: dict[str, object], assets: dict[str, bytes] | None = None,
                    arch: str = "mfq_b200_decoder", extra: dict | None = None, shard_bytes: int | None = None,
                    shard_tensors: int | None = None):
    """Write the checkpoint; with ``shard_bytes`` as ``stem-0000i-of-0000N.mfq`` files (returns their paths)."""
    records = {}
    from .formats import model_graph
    all_assets = {"model_config.json": json.dumps(config).encode(),
                  model_graph.ASSET_NAME: model_graph.to_bytes(model_graph.build_graph(config, tensors.keys(), arch))}
    all_assets.update(assets or {})
    for k, v in all_assets.items():  # assets first: they land in the first shard
        records[ASSET_PREFIX + k] = v
    records.update(tensors)
    header = F.FileHeader(model_arch=arch, extra={"runtime_assets": sorted(all_assets), **(extra or {})})
    if shard_bytes or shard_tensors:
        return F.save_sharded(path, header, records, shard_bytes, shard_tensors)
    F.save(path, header, records)
    return [path]


def load_engine(path, device="cuda", *, native_4bit: bool = False, expert_slots: int | None = None, max_batch: int = 64,
                max_seq_len: int = 8192, tp_rank: int = 0, tp_size: int = 1,
                collective=None, use_graphs: bool = True, kv_budget_bytes: int | None = None,
                yarn_context_extension: float | None = None, mtp_draft_tokens: int = 0, mtp_adaptive: bool = False, mtp_dynamic_depth: bool = False,
                lp_rank: int = 0, lp_size: int = 1, layer_split=None, expert_graphs: bool = False):
    """``.mfq`` -> (engine, tokenizer, config).  ``kv_budget_bytes`` caps the paged KV pool (see ``engine/kv_budget.py``);
    on a GPU it defaults to 90 % of the memory that is free once the weights are resident.  ``yarn_context_extension``
    (> 1) runs the model on that multiple of its trained context with YaRN-scaled rotary frequencies.
    ``mtp_draft_tokens`` (K > 0, only with a checkpoint that carries a ``predictor.*`` head): greedy rows decode by
    draft/verify cycles; ``mtp_adaptive`` parks the cycles while they are slower than plain decoding.
    ``expert_graphs`` (with ``expert_slots``): decode inside CUDA graphs with the experts that are resident and settle
    misses after the step (``LLMEngine.enable_expert_residency_graphs``); without it such a model decodes eagerly."""
    from .engine.llm_engine import LLMEngine
    from .models.moe_decoder import MoeDecoderConfig, MoeDecoderModel, MoeWeights
    from .server.tokenizer import tokenizer_from_assets
    import contextlib
    if Path(path).is_dir():  # a Hugging Face directory served directly: float tensors, transcoded to FP8 on load
        raw, hf_tensors, assets = read_hf_directory(path)
        opened = contextlib.nullcontext(hf_tensors)
    else:
        opened = F.open_mfq(path)
    with opened as store:
        header = None
        if not isinstance(store, dict):
            assets = store.assets()
            header = store.header
            raw = json.loads(assets["model_config.json"])
            from .formats.legacy_names import canonical_view
            store = canonical_view(store)  # old artifacts kept source tensor paths
        if yarn_context_extension and yarn_context_extension > 1.0:
            trained = int((raw.get("rope_scaling") or {}).get("original_max_position") or raw.get("max_position") or 8192)
            raw["rope_scaling"] = dict(raw.get("rope_scaling") or {}, factor=float(yarn_context_extension), original_max_position=trained)
            raw["max_position"] = int(trained * yarn_context_extension)
        if raw.get("kv_lora_rank"):  # latent attention family
            from .models.mla import MlaConfig, MlaModel, mla_weights_from_tensors
            if tp_size != 1:
                raise NotImplementedError("latent-attention checkpoints load on a single rank")
            cfg = MlaConfig(**{k: v for k, v in raw.items() if k in MlaConfig.__dataclass_fields__})
            weights = mla_weights_from_tensors(cfg, store, device)
            model = MlaModel(cfg, weights)
        else:
            fields = {f for f in MoeDecoderConfig.__dataclass_fields__}
            cfg = MoeDecoderConfig(**{k: v for k, v in raw.items() if k in fields})
            weights = MoeWeights.from_tensors(cfg, store, device, tp_rank, tp_size, expert_slots=expert_slots, native_4bit=native_4bit,
                                              lp_rank=lp_rank, lp_size=lp_size, layer_split=layer_split)
            model = MoeDecoderModel(cfg, weights, collective=collective)
    # host-tier experts read the routing on the host every step, which a captured graph cannot do; with
    # ``expert_graphs`` the step translates ids on the device instead and the engine settles misses afterwards
    num_pages = None
    if kv_budget_bytes is None and str(device).startswith("cuda"):
        from .engine.kv_budget import device_budget
        kv_budget_bytes = device_budget(device)
    if kv_budget_bytes is not None:
        from .engine.kv_budget import plan
        has_head = getattr(weights, "mtp", None) is not None
        num_pages = plan(budget_bytes=kv_budget_bytes, layers=model.local_layers + int(has_head), kv_heads=model.hk, head_dim=cfg.head_dim,
                         max_batch=max_batch, max_seq_len=max_seq_len).num_pages
    engine = LLMEngine(model, max_batch=max_batch, max_seq_len=max_seq_len, device=device, num_pages=num_pages,
                       use_graphs=use_graphs and (expert_slots is None or expert_graphs),
                       mtp_draft_tokens=mtp_draft_tokens if getattr(weights, "mtp", None) is not None else 0,
                       mtp_adaptive=mtp_adaptive and tp_size == 1, mtp_dynamic_depth=mtp_dynamic_depth and tp_size == 1)  # ranks time their steps separately: they would
    #                                                                    park at different moments and fall out of lockstep
    if expert_slots is not None and expert_graphs and not engine.enable_expert_residency_graphs():
        engine.use_graphs = engine.use_graphs and not (hasattr(model, "residencies") and model.residencies())
    # what the checkpoint says about itself, for the server's sampling-profile resolution
    engine.checkpoint_meta = {
        "path": str(path), "header_extra": dict(getattr(header, "extra", None) or {}),
        "architecture": raw.get("model_type") or raw.get("family") or getattr(header, "model_arch", "") or "",
        "assets": {k: v for k, v in assets.items() if k == "hf/generation_config.json"}}
    tokenizer = tokenizer_from_assets(assets, cfg.vocab_size)
    # structured output needs the vocabulary's byte strings; resolved on the first request that asks for it
    engine.set_token_bytes(lambda: tokenizer.token_bytes(cfg.vocab_size), tokenizer.stop_ids)
    return engine, tokenizer, cfg
