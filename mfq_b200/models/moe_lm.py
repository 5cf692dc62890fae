"""Mixture-of-experts decoder with per-expert-projection mixed formats (CPU / reference execution path).

``MoeLM`` is the plain-PyTorch restatement of the MoE model family: GQA attention with RoPE, RMSNorm, a softmax
(or sigmoid) router with top-k selection, SwiGLU experts and an optional shared expert.  It runs on fp32 weights
that are either the original bf16 values or the *dequantized* per-expert mixed-format weights, which makes it the
oracle for quantization quality (KLD / top-1 agreement against the bf16 model) and for the GPU MoE kernels.

``quantize_moe_checkpoint`` applies the seeded balanced allocation of families to every routed expert projection
(gate / up / down separately, the rule of ``mfq/tools/quantize_hf_to_mfq.py:2598-2619``) and returns tensors under
the canonical checkpoint names (``mfq/architectures/tensor_schema.py:551-596``), ready for ``formats.save``.
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import numpy as np
import torch

from .. import formats as F
from ..quantize import (DEFAULT_MIX_SEED, balanced_expert_mix, parse_profiles, quantize_expertwise, quantize_fp8_block,
                        quantize_nint)


@dataclass
class MoeConfig:
    vocab_size: int = 1024
    hidden_size: int = 256
    num_layers: int = 2
    num_heads: int = 4
    num_kv_heads: int = 2
    head_dim: int = 64
    rope_theta: float = 1e6
    rms_eps: float = 1e-6
    num_experts: int = 8
    top_k: int = 2
    moe_intermediate: int = 128
    shared_intermediate: int = 0  # 0 = no shared expert
    router: str = "softmax"  # or "sigmoid"
    norm_topk: bool = True
    name: str = "tiny-moe"


def init_weights(cfg: MoeConfig, seed: int = 0, std: float = 0.02) -> dict[str, torch.Tensor]:
    """Random N(0, std) bf16-representable weights under canonical tensor names."""
    g = torch.Generator().manual_seed(seed)

    def rnd(*shape):
        return (torch.randn(shape, generator=g) * std).to(torch.bfloat16).float()

    h, d = cfg.hidden_size, cfg.head_dim
    w = {"model.token_embedding.weight": rnd(cfg.vocab_size, h), "model.output_norm.weight": torch.ones(h),
         "model.output.weight": rnd(cfg.vocab_size, h)}
    for i in range(cfg.num_layers):
        p = f"model.block.{i}."
        w[p + "attention.norm.weight"] = torch.ones(h)
        w[p + "attention.query.weight"] = rnd(cfg.num_heads * d, h)
        w[p + "attention.key.weight"] = rnd(cfg.num_kv_heads * d, h)
        w[p + "attention.value.weight"] = rnd(cfg.num_kv_heads * d, h)
        w[p + "attention.output.weight"] = rnd(h, cfg.num_heads * d)
        w[p + "mlp.norm.weight"] = torch.ones(h)
        w[p + "mlp.router.weight"] = rnd(cfg.num_experts, h)
        w[p + "mlp.experts.gate.weight"] = rnd(cfg.num_experts, cfg.moe_intermediate, h)
        w[p + "mlp.experts.up.weight"] = rnd(cfg.num_experts, cfg.moe_intermediate, h)
        w[p + "mlp.experts.down.weight"] = rnd(cfg.num_experts, h, cfg.moe_intermediate)
        if cfg.shared_intermediate:
            w[p + "mlp.shared_expert.gate.weight"] = rnd(cfg.shared_intermediate, h)
            w[p + "mlp.shared_expert.up.weight"] = rnd(cfg.shared_intermediate, h)
            w[p + "mlp.shared_expert.down.weight"] = rnd(h, cfg.shared_intermediate)
    return w


def quantize_moe_checkpoint(weights: dict[str, torch.Tensor], expert_mix: str = "NINT4,NVQ3,MXFP4",
                            seed: int = DEFAULT_MIX_SEED, dense: str = "bf16") -> dict[str, object]:
    """Per-expert-projection mixed quantization of the routed experts; dense tensors stay bf16 (or NINT / FP8)."""
    profiles = parse_profiles(expert_mix)
    out: dict[str, object] = {}
    for name, t in weights.items():
        a = t.numpy().astype(np.float32)
        if ".mlp.experts." in name and a.ndim == 3:
            assign = balanced_expert_mix(name, a.shape[0], len(profiles), seed)
            out[name] = quantize_expertwise(a, assign, profiles)
        elif a.ndim == 2 and dense == "nint4" and "norm" not in name and "router" not in name:
            out[name] = quantize_nint(a, F.NintSpec())
        elif a.ndim == 2 and dense == "fp8" and "norm" not in name and "router" not in name and a.shape[1] % 128 == 0:
            out[name] = quantize_fp8_block(a)
        else:
            out[name] = F.to_bf16(a)
    return out


def dequantize_checkpoint(tensors: dict[str, object]) -> dict[str, torch.Tensor]:
    return {name: torch.from_numpy(np.ascontiguousarray(F.dequantize(t))).float() for name, t in tensors.items()
            if not isinstance(t, (bytes, bytearray))}


def _rms(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * w


def _rope(x: torch.Tensor, pos: torch.Tensor, theta: float) -> torch.Tensor:
    d = x.shape[-1]
    half = d // 2
    inv = torch.exp2(-math.log2(theta) * (2 * torch.arange(half, dtype=torch.float32)) / d)
    ang = pos.float()[:, None] * inv[None]
    c, s = ang.cos()[:, None], ang.sin()[:, None]
    a, b = x[..., :half], x[..., half:]
    return torch.cat([a * c - b * s, b * c + a * s], -1)


def route(logits: torch.Tensor, cfg: MoeConfig) -> tuple[torch.Tensor, torch.Tensor]:
    """Top-k expert ids and normalized weights per token (softmax-then-top-k, or sigmoid scores)."""
    scores = torch.softmax(logits.float(), -1) if cfg.router == "softmax" else torch.sigmoid(logits.float())
    w, idx = torch.topk(scores, cfg.top_k, dim=-1)
    if cfg.norm_topk:
        w = w / w.sum(-1, keepdim=True).clamp_min(1e-20)
    return idx, w


class MoeLM:
    """fp32 forward with a plain KV list (no paging): prefill a prompt, then decode token by token."""

    def __init__(self, cfg: MoeConfig, weights: dict[str, torch.Tensor], observer=None, reap_observer=None,
                 input_transform=None) -> None:
        """``observer(name, x, y)`` (optional) sees input and output of every named 2-D projection: the hook the
        importance-matrix collection uses.  ``reap_observer(name, route_weights, y)`` (optional) sees every routed
        expert's outputs and the router weights of its tokens (``name`` = ``<down tensor>#<expert>``)."""
        self.cfg, self.w = cfg, weights
        self.observer = observer
        self.reap_observer = reap_observer
        # ``input_transform(x)`` (optional) replaces the input of every named 2-D projection, e.g. by its NINT8-1
        # reconstruction, to measure a checkpoint under the activation rounding of an int8-activation runtime
        self.input_transform = input_transform
        self.k_cache: list[torch.Tensor] = []
        self.v_cache: list[torch.Tensor] = []

    def _lin(self, name: str, x: torch.Tensor) -> torch.Tensor:
        if self.input_transform is not None:
            x = self.input_transform(x).to(x.dtype)
        y = x @ self.w[name].T
        if self.observer is not None:
            self.observer(name, x, y)
        return y

    def reset(self) -> None:
        self.k_cache, self.v_cache = [], []

    def _moe(self, x: torch.Tensor, p: str) -> torch.Tensor:
        cfg, w = self.cfg, self.w
        idx, wt = route(x @ w[p + "mlp.router.weight"].T, cfg)
        out = torch.zeros_like(x)
        gate, up, down = w[p + "mlp.experts.gate.weight"], w[p + "mlp.experts.up.weight"], w[p + "mlp.experts.down.weight"]
        for e in idx.unique().tolist():
            tok, slot = (idx == e).nonzero(as_tuple=True)
            xe = x[tok]
            he = torch.nn.functional.silu(xe @ gate[e].T) * (xe @ up[e].T)
            if self.observer is not None:  # per-expert statistics: "<tensor>#<expert>", inputs only
                self.observer(f"{p}mlp.experts.gate.weight#{e}", xe, None)
                self.observer(f"{p}mlp.experts.up.weight#{e}", xe, None)
                self.observer(f"{p}mlp.experts.down.weight#{e}", he, None)
            ye = he @ down[e].T
            if self.reap_observer is not None:
                self.reap_observer(f"{p}mlp.experts.down.weight#{e}", wt[tok, slot], ye)
            out.index_add_(0, tok, ye * wt[tok, slot][:, None])
        if cfg.shared_intermediate:
            hs = torch.nn.functional.silu(self._lin(p + "mlp.shared_expert.gate.weight", x)) * self._lin(p + "mlp.shared_expert.up.weight", x)
            out = out + self._lin(p + "mlp.shared_expert.down.weight", hs)
        return out

    def forward(self, ids: torch.Tensor) -> torch.Tensor:
        """Append ``ids`` to the sequence; returns fp32 logits ``[len(ids), vocab]``."""
        cfg, w = self.cfg, self.w
        t = ids.numel()
        start = self.k_cache[0].shape[0] if self.k_cache else 0
        pos = torch.arange(start, start + t)
        x = w["model.token_embedding.weight"][ids.long()]
        g = cfg.num_heads // cfg.num_kv_heads
        for i in range(cfg.num_layers):
            p = f"model.block.{i}."
            h = _rms(x, w[p + "attention.norm.weight"], cfg.rms_eps)
            q = _rope(self._lin(p + "attention.query.weight", h).view(t, cfg.num_heads, cfg.head_dim), pos, cfg.rope_theta)
            k = _rope(self._lin(p + "attention.key.weight", h).view(t, cfg.num_kv_heads, cfg.head_dim), pos, cfg.rope_theta)
            v = self._lin(p + "attention.value.weight", h).view(t, cfg.num_kv_heads, cfg.head_dim)
            if len(self.k_cache) <= i:
                self.k_cache.append(k)
                self.v_cache.append(v)
            else:
                self.k_cache[i] = torch.cat([self.k_cache[i], k])
                self.v_cache[i] = torch.cat([self.v_cache[i], v])
            kk = self.k_cache[i].repeat_interleave(g, 1)
            vv = self.v_cache[i].repeat_interleave(g, 1)
            s = torch.einsum("qhd,khd->hqk", q, kk) / math.sqrt(cfg.head_dim)
            mask = torch.arange(kk.shape[0])[None, :] > pos[:, None]
            s = s.masked_fill(mask[None], float("-inf"))
            a = torch.einsum("hqk,khd->qhd", torch.softmax(s, -1), vv).reshape(t, -1)
            x = x + self._lin(p + "attention.output.weight", a)
            x = x + self._moe(_rms(x, w[p + "mlp.norm.weight"], cfg.rms_eps), p)
        x = _rms(x, w["model.output_norm.weight"], cfg.rms_eps)
        return self._lin("model.output.weight", x)
