"""Read-only analyses of catalogued checkpoints and of the running service, for the control API.

* :func:`checkpoint_analysis` -- what a packed checkpoint is made of: bytes and tensor counts per family, bits per weight
  per tensor group (attention / dense MLP / routed experts / shared experts / embeddings / head / predictor / norms), the
  largest tensors, shard count.  Element counts come from the tensors' own payload headers for checkpoints up to 256 MB
  and from the model configuration for larger ones, so that a multi-gigabyte file is never decoded for a listing.
* :func:`model_parameters` -- parameter counts per group from the model configuration, total and ACTIVE per token (a
  mixture-of-experts model touches ``top_k`` of its routed experts).
* :func:`model_memory` -- device memory a deployment needs: resident weights (per rank under tensor / expert parallelism),
  the paged FP8 KV cache for a batch and context (16-token pages, two code bytes per head dimension and 8 bytes of
  multipliers per token, head and layer), recurrent state of hybrid layers, and the fixed workspaces.
* :func:`serving_stats` -- request counts, token totals and latency / throughput quantiles estimated from the metrics
  histograms of the running service.

Reference: ``mfq/server/services/{checkpoint_analysis,model_parameters,model_memory,serving_stats}.py``.
"""

from __future__ import annotations

import json
import math
from pathlib import Path

GROUPS = (("predictor", "predictor."), ("routed_experts", ".mlp.experts."), ("shared_experts", ".mlp.shared_expert"),
          ("router", ".mlp.router"), ("attention", ".attention."), ("linear_attention", ".linear_attention."),
          ("dense_mlp", ".mlp."), ("embeddings", "token_embedding"), ("head", "model.output.weight"), ("norms", "norm"))


def group_of(name: str) -> str:
    for label, piece in GROUPS:
        if piece in name:
            return label
    return "other"


def _weights_of(store, name: str) -> int | None:
    """Logical element count of a stored tensor, from its self-describing payload header where that is cheap."""
    from ..formats import unpack_tensor
    dtype = store.dtype(name)
    try:
        t = unpack_tensor(store.records[name].dtype, store.raw(name))
    except Exception:
        return None
    shape = getattr(t, "shape", None)
    if shape is None:
        return None
    return int(math.prod(int(s) for s in shape)) if dtype != "BLOB" else None


def checkpoint_analysis(path, *, count_weights: bool | None = None, largest: int = 8, decode_limit: int = 256 << 20) -> dict:
    """``count_weights``: read element counts out of every tensor's payload (None: only for checkpoints of at most
    ``decode_limit`` bytes; larger ones take the per-group counts of their model configuration instead)."""
    from ..formats import ASSET_PREFIX, open_mfq
    with open_mfq(path) as store:
        if count_weights is None:
            count_weights = sum(r.nbytes for r in store.records.values()) <= decode_limit
        by_dtype: dict[str, dict] = {}
        by_group: dict[str, dict] = {}
        tensors = []
        for name, rec in store.records.items():
            if name.startswith(ASSET_PREFIX):
                continue
            d = store.dtype(name)
            a = by_dtype.setdefault(d, {"tensors": 0, "bytes": 0})
            a["tensors"] += 1
            a["bytes"] += rec.nbytes
            g = by_group.setdefault(group_of(name), {"tensors": 0, "bytes": 0, "weights": 0})
            g["tensors"] += 1
            g["bytes"] += rec.nbytes
            w = _weights_of(store, name) if count_weights else None
            if w:
                g["weights"] += w
            tensors.append((rec.nbytes, name, d, w))
        assets = store.assets()
        cfg = json.loads(assets["model_config.json"]) if "model_config.json" in assets else {}
        if not count_weights and cfg:
            for label, n in model_parameters(cfg)["groups"].items():
                if label in by_group:
                    by_group[label]["weights"] = n
        for g in by_group.values():
            g["bits_per_weight"] = round(8.0 * g["bytes"] / g["weights"], 3) if g["weights"] else None
        total_bytes = sum(v["bytes"] for v in by_dtype.values())
        total_weights = sum(v["weights"] for v in by_group.values())
        tensors.sort(reverse=True)
        return {"path": str(path), "arch": store.header.model_arch, "format_version": store.header.version,
                "shards": len({r.file_index for r in store.records.values()}), "tensors": len(tensors), "bytes": total_bytes,
                "weights": total_weights or None,
                "bits_per_weight": round(8.0 * total_bytes / total_weights, 3) if total_weights else None,
                "by_dtype": by_dtype, "by_group": by_group,
                "largest": [{"name": n, "dtype": d, "bytes": b, "weights": w} for b, n, d, w in tensors[:largest]],
                "assets": sorted(assets), "config": {k: cfg[k] for k in sorted(cfg) if isinstance(cfg[k], (int, float, str, bool))},
                "quantization": (store.header.extra or {}).get("quantization")}


def _cfg_int(cfg: dict, *names, default: int = 0) -> int:
    for n in names:
        if cfg.get(n) is not None:
            return int(cfg[n])
    return default


def model_parameters(cfg: dict) -> dict:
    """Counts from a model configuration (canonical keys of ``model_config.json``; Hugging Face spellings accepted)."""
    h = _cfg_int(cfg, "hidden_size")
    layers = _cfg_int(cfg, "num_layers", "num_hidden_layers")
    hq = _cfg_int(cfg, "num_heads", "num_attention_heads")
    hk = _cfg_int(cfg, "num_kv_heads", "num_key_value_heads", default=hq)
    d = _cfg_int(cfg, "head_dim", default=h // max(1, hq))
    vocab = _cfg_int(cfg, "vocab_size")
    inter = _cfg_int(cfg, "intermediate_size")
    experts = _cfg_int(cfg, "num_experts", "n_routed_experts")
    top_k = _cfg_int(cfg, "top_k", "num_experts_per_tok")
    moe_inter = _cfg_int(cfg, "moe_intermediate", "moe_intermediate_size")
    shared = _cfg_int(cfg, "shared_intermediate", "shared_expert_intermediate_size")
    full_every = _cfg_int(cfg, "full_attention_interval", default=1)  # hybrid models: every n-th layer is full attention
    attn_layers = layers if full_every <= 1 else layers // full_every
    attn = attn_layers * (h * (hq + 2 * hk) * d + hq * d * h)
    linear_layers = layers - attn_layers
    lin_k, lin_v = _cfg_int(cfg, "linear_num_key_heads"), _cfg_int(cfg, "linear_num_value_heads")
    lin_dk, lin_dv = _cfg_int(cfg, "linear_key_head_dim", default=128), _cfg_int(cfg, "linear_value_head_dim", default=128)
    linear = linear_layers * (h * (2 * lin_k * lin_dk + 2 * lin_v * lin_dv) + lin_v * lin_dv * h) if linear_layers and lin_v else 0
    dense_mlp = layers * 3 * h * inter if inter and not experts else 0
    routed = layers * experts * 3 * h * moe_inter if experts else 0
    routed_active = layers * top_k * 3 * h * moe_inter if experts else 0
    shared_p = layers * 3 * h * shared if shared else 0
    router = layers * experts * h if experts else 0
    emb = vocab * h
    head = 0 if cfg.get("tie_word_embeddings") else vocab * h
    norms = layers * 2 * h + h
    groups = {"attention": attn, "linear_attention": linear, "dense_mlp": dense_mlp, "routed_experts": routed, "shared_experts": shared_p,
              "router": router, "embeddings": emb, "head": head, "norms": norms}
    total = sum(groups.values())
    active = total - routed + routed_active
    return {"groups": {k: v for k, v in groups.items() if v}, "total": total, "active_per_token": active,
            "experts": experts or None, "top_k": top_k or None, "layers": layers, "attention_layers": attn_layers}


def model_memory(cfg: dict, weight_bytes: int, *, batch: int = 1, context: int = 4096, tensor_parallel: int = 1,
                 expert_bytes: int = 0, workspace_bytes: int = (64 << 20) + (16 << 22) + (8 << 20)) -> dict:
    """Bytes per GPU.  ``weight_bytes``: the checkpoint's tensor bytes; ``expert_bytes``: the share of them in routed
    experts (split over ranks by expert, everything else by tensor parallelism except replicated norms / router)."""
    from ..engine.kv_budget import PAGE_TOKENS, page_bytes
    p = model_parameters(cfg)
    hk = max(1, _cfg_int(cfg, "num_kv_heads", "num_key_value_heads", default=_cfg_int(cfg, "num_heads", "num_attention_heads")))
    hq = _cfg_int(cfg, "num_heads", "num_attention_heads")
    d = _cfg_int(cfg, "head_dim", default=_cfg_int(cfg, "hidden_size") // max(1, hq))
    tp = max(1, int(tensor_parallel))
    pages = batch * math.ceil(context / PAGE_TOKENS) + 1
    kv = pages * page_bytes(p["attention_layers"], max(1, hk // tp), d)
    lin_v = _cfg_int(cfg, "linear_num_value_heads")
    state = 0
    if lin_v:
        lin_layers = p["layers"] - p["attention_layers"]
        dk, dv = _cfg_int(cfg, "linear_key_head_dim", default=128), _cfg_int(cfg, "linear_value_head_dim", default=128)
        state = batch * lin_layers * max(1, lin_v // tp) * dk * dv * 4
    weights = (weight_bytes - expert_bytes) // tp + expert_bytes // tp
    total = weights + kv + state + workspace_bytes
    return {"per_gpu": {"weights": weights, "kv_cache": kv, "recurrent_state": state, "workspaces": workspace_bytes, "total": total},
            "gpus": tp, "batch": batch, "context": context, "kv_bytes_per_token": kv // max(1, batch * context),
            "fits_180gb": total <= 180 * 10 ** 9}


def _quantile(buckets, counts, total: int, q: float) -> float | None:
    if not total:
        return None
    want, prev_le, prev_c = q * total, 0.0, 0
    for le, c in zip(buckets, counts):
        if c >= want:
            if math.isinf(le):
                return prev_le
            span = c - prev_c
            return prev_le + (le - prev_le) * ((want - prev_c) / span if span else 1.0)
        prev_le, prev_c = (0.0 if math.isinf(le) else le), c
    return prev_le


def serving_stats(metrics) -> dict:
    """Per model: counters as they are, histograms as count / mean / p50 / p95 (linear inside a bucket)."""
    from .metrics import _BUCKETS
    out: dict[str, dict] = {}
    with metrics._lock:
        counters = dict(metrics._counters)
        hists = {k: {"sum": v["sum"], "count": v["count"], "b": list(v["b"])} for k, v in metrics._hist.items()}
    for (name, model, _instance, extra), value in counters.items():
        m = out.setdefault(model, {"counters": {}, "histograms": {}})
        label = name + ("{" + ",".join(f"{k}={v}" for k, v in extra) + "}" if extra else "")
        m["counters"][label] = m["counters"].get(label, 0.0) + value
    for (name, model, _instance, _extra), h in hists.items():
        m = out.setdefault(model, {"counters": {}, "histograms": {}})
        agg = m["histograms"].setdefault(name, {"sum": 0.0, "count": 0, "b": [0] * len(_BUCKETS[name])})
        agg["sum"] += h["sum"]
        agg["count"] += h["count"]
        agg["b"] = [a + b for a, b in zip(agg["b"], h["b"])]
    for m in out.values():
        for name, agg in list(m["histograms"].items()):
            n = agg["count"]
            m["histograms"][name] = {"count": n, "mean": agg["sum"] / n if n else None,
                                     "p50": _quantile(_BUCKETS[name], agg["b"], n, 0.5), "p95": _quantile(_BUCKETS[name], agg["b"], n, 0.95)}
    return {"models": out}


def analyse_artifact(artifact, *, batch: int = 1, context: int = 4096, tensor_parallel: int = 1) -> dict:
    """Everything the catalog routes report for one entry (packed checkpoints: full analysis; others: what is known)."""
    if artifact.kind != "mfq":
        cfg = {}
        p = Path(artifact.path)
        if artifact.kind == "hf" and (p / "config.json").exists():
            cfg = json.loads((p / "config.json").read_text())
            cfg = cfg.get("text_config", cfg)
        out = {"id": artifact.id, "kind": artifact.kind, "bytes": artifact.bytes}
        if cfg:
            out["parameters"] = model_parameters(cfg)
            out["memory"] = model_memory(cfg, artifact.bytes, batch=batch, context=context, tensor_parallel=tensor_parallel)
        return out
    a = checkpoint_analysis(artifact.path)
    from ..formats import open_mfq
    with open_mfq(artifact.path) as store:
        assets = store.assets()
        cfg = json.loads(assets["model_config.json"]) if "model_config.json" in assets else {}
    expert_bytes = a["by_group"].get("routed_experts", {}).get("bytes", 0)
    return {"id": artifact.id, "kind": "mfq", "analysis": a, "parameters": model_parameters(cfg) if cfg else None,
            "memory": model_memory(cfg, a["bytes"], batch=batch, context=context, tensor_parallel=tensor_parallel,
                                   expert_bytes=expert_bytes) if cfg else None}
