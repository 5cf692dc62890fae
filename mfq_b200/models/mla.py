"""Multi-head latent attention (DeepSeek-V3 style) on top of the MoE decoder.

Projections: ``q = q_b(rmsnorm(q_a(x)))`` (or one ``q_b`` when the query is not compressed), ``kv_a(x)`` gives the shared
latent ``c`` (``kv_lora_rank``) and one rotary key part for all heads, ``kv_b(rmsnorm(c))`` expands the latent into a
non-rotary key part and a value per head.  A head's score is ``q_nope . k_nope + q_rope . k_rope`` scaled by
``1 / sqrt(nope + rope)``.

Execution here is the direct (non-absorbed) form on the existing 256-wide attention kernels: every head's query and key
are laid out as ``[rope | nope | 0]`` (64 + 128 + 64 zeros = 256; the rotary part first, because the rope / page-write
kernel rotates the leading dims) and its value as ``[v | 0]``; a consistent permutation plus zero padding leaves every dot
product unchanged, and the first ``v_head_dim`` columns of the attention output are the result.  The paged cache therefore
holds expanded per-head keys and values (FP8), not the latent: this runs the model family correctly on the GPU kernels
that exist, at a cache cost of ``2 * 256`` bytes per head and token instead of ``kv_lora_rank + rope``.  The
latent cache with weight-absorbed decode is the form to build next.  Reference: ``cpp_runtime/models/deepseek_v4`` /
``glm_dsa`` graphs and ``mfq/kernels/cuda/deepseek_v4_attention.cu``.
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import torch

from .. import ops
from ..ops import reference as ref
from .llama import Fp8Linear, StepBuffers
from .moe_decoder import MoeDecoderConfig, MoeDecoderModel, MoeFfn, MoeLayer, MoeWeights

PADDED_HEAD = 256


@dataclass
class MlaConfig(MoeDecoderConfig):
    q_lora_rank: int = 1536  # 0: queries are projected directly
    kv_lora_rank: int = 512
    qk_nope_head_dim: int = 128
    qk_rope_head_dim: int = 64
    v_head_dim: int = 128
    absorbed: bool = False  # latent cache + weight-absorbed attention (GPU kernels need latent 512 + rotary 64)
    name: str = "mla-moe-fp8"

    def __post_init__(self):
        if self.qk_nope_head_dim + self.qk_rope_head_dim > PADDED_HEAD or self.v_head_dim > PADDED_HEAD:
            raise ValueError("head parts do not fit the 256-wide attention kernels")
        if self.absorbed:
            # the cache holds one shared row per token: [rotary key part | normalised latent]
            if (self.kv_lora_rank + self.qk_rope_head_dim) % 64:
                raise ValueError("latent + rotary width must be a multiple of 64 (cache chunking)")
            self.head_dim = self.kv_lora_rank + self.qk_rope_head_dim
            self.num_kv_heads = 1
            return
        # the cache and the attention kernels see plain multi-head attention with padded 256-wide heads
        self.head_dim = PADDED_HEAD
        self.num_kv_heads = self.num_heads

    @classmethod
    def tiny(cls) -> "MlaConfig":
        return cls(vocab_size=1024, hidden_size=256, intermediate_size=512, num_layers=3, num_heads=2, num_kv_heads=2,
                   head_dim=PADDED_HEAD, rope_theta=1e4, rms_eps=1e-6, num_experts=8, top_k=2, moe_intermediate=128,
                   shared_intermediate=128, router="sigmoid", n_group=2, topk_group=1, routed_scale=2.5, first_dense_layers=1,
                   q_lora_rank=128, kv_lora_rank=128, name="tiny-mla-moe-fp8")

    @classmethod
    def v3_style(cls, num_layers: int = 61) -> "MlaConfig":
        """The DeepSeek-V3 geometry (671B with 61 layers); fewer layers give a model of the same widths that fits."""
        return cls(vocab_size=129280, hidden_size=7168, intermediate_size=18432, num_layers=num_layers, num_heads=128,
                   num_kv_heads=128, head_dim=PADDED_HEAD, rope_theta=1e4, rms_eps=1e-6, num_experts=256, top_k=8,
                   moe_intermediate=2048, shared_intermediate=2048, router="sigmoid", n_group=8, topk_group=4,
                   routed_scale=2.5, first_dense_layers=min(3, num_layers), name=f"v3-style-mla-moe-{num_layers}l")


@dataclass
class MlaWeights:
    q_a: Fp8Linear | None  # [q_lora, H]
    q_a_norm: torch.Tensor | None
    q_b: Fp8Linear  # [Hq * (nope + rope), q_lora or H]
    kv_a: Fp8Linear  # [kv_lora + rope, H]
    kv_a_norm: torch.Tensor
    kv_b: Fp8Linear  # [Hq * (nope + v), kv_lora]


@dataclass
class MlaLayer(MoeLayer):
    mla: MlaWeights | None = None


class MlaModel(MoeDecoderModel):
    """:class:`MoeDecoderModel` whose attention blocks are latent attention wherever the layer carries ``mla`` weights."""

    def __init__(self, cfg: MlaConfig, weights, collective=None) -> None:
        super().__init__(cfg, weights, collective=collective)
        if self.tp != 1:
            raise NotImplementedError("latent attention is single-rank for now")
        self.sm_scale = 1.0 / math.sqrt(cfg.qk_nope_head_dim + cfg.qk_rope_head_dim)
        if self.rope_scaling is not None:
            self.sm_scale *= self.rope_scaling.softmax_scale_factor
        self.attn_rot = cfg.qk_rope_head_dim
        if cfg.absorbed:
            self.hk = 1  # all query heads attend to the one latent row per token
            self._absorb: dict[int, tuple[torch.Tensor, torch.Tensor]] = {}

    def _absorbed_weights(self, layer):
        """kv_b split per head into the key part ``[Hq, nope, latent]`` and the value part ``[Hq, v, latent]``."""
        key = id(layer)
        if key not in self._absorb:
            cfg = self.cfg
            wkv = layer.mla.kv_b.dequant().float().view(self.hq, cfg.qk_nope_head_dim + cfg.v_head_dim, cfg.kv_lora_rank)
            self._absorb[key] = (wkv[:, : cfg.qk_nope_head_dim].contiguous(), wkv[:, cfg.qk_nope_head_dim :].contiguous())
        return self._absorb[key]

    def _mla_absorbed(self, h, layer, kv, step: StepBuffers, prefill: bool):
        """Weight-absorbed form: ``q_nope . (W_k c) = (W_k^T q_nope) . c`` and ``sum_s p_s W_v c_s = W_v sum_s p_s c_s``,
        so keys and values never exist per head: the cache keeps ``[k_rope | c]`` once per token (``kv_lora + rope``
        values instead of ``2 * Hq * 256``), queries are mapped into the latent space, attention runs as Hq query heads
        over one shared key/value row, and the latent output is expanded by ``W_v`` afterwards."""
        if h.is_cuda:
            return self._mla_absorbed_gpu(h, layer, kv, step, prefill)
        cfg, m = self.cfg, layer.mla
        nope, rope, vd, hq, lat = cfg.qk_nope_head_dim, cfg.qk_rope_head_dim, cfg.v_head_dim, self.hq, cfg.kv_lora_rank
        t = h.shape[0]
        xq, xs = self._norm_quant(h, layer.attn_norm)
        q = (m.q_b(*self._norm_quant(m.q_a(xq, xs), m.q_a_norm)) if m.q_a is not None else m.q_b(xq, xs)).view(t, hq, nope + rope)
        ckv = m.kv_a(xq, xs)
        c_n = ref.rmsnorm(ckv[:, :lat].contiguous(), m.kv_a_norm, cfg.rms_eps)  # bf16 [T, latent]
        wk, wv = self._absorbed_weights(layer)
        q_abs = torch.einsum("thn,hnl->thl", q[:, :, :nope].float(), wk).to(torch.bfloat16)
        d = rope + lat
        qkv = torch.zeros((t, hq + 2, d), dtype=torch.bfloat16)
        qkv[:, :hq, :rope] = q[:, :, nope:]
        qkv[:, :hq, rope:] = q_abs
        qkv[:, hq, :rope] = ckv[:, lat:]
        qkv[:, hq, rope:] = c_n
        qkv[:, hq + 1, :lat] = c_n  # value row = the latent (the cache class keeps keys and values the same width)
        o_lat = self._attention(qkv.view(t, (hq + 2) * d), kv, step, prefill).view(t, hq, d)[:, :, :lat]
        return torch.einsum("thl,hvl->thv", o_lat.float(), wv).to(torch.bfloat16).reshape(t, hq * vd)

    def _mla_absorbed_gpu(self, h, layer, kv, step: StepBuffers, prefill: bool):
        """The same on the GPU.  Every token's ``[k_rope | latent]`` row goes to the FP8 latent cache; decode steps run
        the shared-row attention kernel over it (``ops/mla.py``) between two small per-head products (``W_k^T q`` in,
        ``W_v o`` out); a prefill chunk attends to itself in the direct per-head form on the 256-wide prefill kernel
        (keys and values expanded from the chunk's own latents, never stored)."""
        from ..ops import mla as mla_ops
        cfg, m = self.cfg, layer.mla
        nope, rope, vd, hq, lat = cfg.qk_nope_head_dim, cfg.qk_rope_head_dim, cfg.v_head_dim, self.hq, cfg.kv_lora_rank
        if lat != mla_ops.LATENT or rope + lat != mla_ops.ROW_WIDTH:
            raise NotImplementedError("the latent-cache kernels are built for a 512-wide latent and a 64-wide rotary part")
        t = h.shape[0]
        xq, xs = self._norm_quant(h, layer.attn_norm)
        q = (m.q_b(*self._norm_quant(m.q_a(xq, xs), m.q_a_norm)) if m.q_a is not None else m.q_b(xq, xs)).view(t, hq, nope + rope)
        ckv = m.kv_a(xq, xs)
        c_n = ops.rmsnorm_quant(ckv[:, :lat].contiguous(), m.kv_a_norm, cfg.rms_eps, want_q=False, want_y=True)[2]
        k_rope = ref.rope(ckv[:, None, lat:], step.positions, cfg.rope_theta, rope, self.rope_scaling)[:, 0]
        q_rope = ref.rope(q[:, :, nope:], step.positions, cfg.rope_theta, rope, self.rope_scaling)
        mla_ops.latent_write(torch.cat([k_rope, c_n], 1), step.slots, kv)
        if prefill:
            past = step.past_len
            rows_k, rows_c = k_rope, c_n
            if past > 0:
                # A chunk after cached tokens: the past rows come back from the latent cache (the FP8 values that decode
                # steps will read) and their per-head keys and values are expanded again -- the cache never holds them.
                from ..engine.kv_cache import k_logical
                pages = step.block_table[0][: (past + kv.page_size - 1) // kv.page_size].long()
                cached = k_logical(kv.k[pages]).float() * kv.k_scale[pages][..., None]  # [pages, 1, 16, 576]
                cached = cached.reshape(-1, rope + lat)[:past].to(torch.bfloat16)
                rows_k = torch.cat([cached[:, :rope], k_rope], 0)
                rows_c = torch.cat([cached[:, rope:], c_n], 0)
            tk = rows_c.shape[0]
            kvb = m.kv_b(*self._quant(rows_c.contiguous())).view(tk, hq, nope + vd)
            qh = torch.zeros((t, hq, PADDED_HEAD), dtype=torch.bfloat16, device=h.device)
            kh = torch.zeros((tk, hq, PADDED_HEAD), dtype=torch.bfloat16, device=h.device)
            vh = torch.zeros_like(kh)
            qh[:, :, :rope], qh[:, :, rope : rope + nope] = q_rope, q[:, :, :nope]
            kh[:, :, :rope], kh[:, :, rope : rope + nope] = rows_k[:, None, :], kvb[:, :, :nope]
            vh[:, :, :vd] = kvb[:, :, nope:]
            if past > 0:
                o = ops.kernels.attn_prefill_bf16(qh, kh, vh, self.sm_scale)
            else:
                o = ops.attn_prefill(qh, kh, vh, step.cu_seqlens, self.sm_scale)
            return o.view(t, hq, PADDED_HEAD)[:, :, :vd].reshape(t, hq * vd)
        block_table, seq_lens = step.block_table, step.seq_lens
        if step.q_len != 1:
            # A window of w query tokens per sequence (speculative verification): every window position becomes a row
            # of its own over the same pages, seeing the context up to itself -- the window's latent rows are in the
            # cache already, so causality is a matter of row lengths.
            w = step.q_len
            back = torch.arange(w - 1, -1, -1, dtype=seq_lens.dtype, device=seq_lens.device)
            seq_lens = (seq_lens[:, None] - back[None, :]).reshape(-1).contiguous()
            block_table = block_table.repeat_interleave(w, 0).contiguous()
        key = ("bf16", id(layer))
        if key not in self._absorb:
            wk, wv = self._absorbed_weights(layer)
            self._absorb[key] = (wk.to(torch.bfloat16).contiguous(), wv.transpose(1, 2).to(torch.bfloat16).contiguous())
        wk, wv_t = self._absorb[key]  # [Hq, nope, latent], [Hq, latent, v]
        q_abs = torch.bmm(q[:, :, :nope].transpose(0, 1), wk).transpose(0, 1)  # [T, Hq, latent]
        o_lat = mla_ops.decode(torch.cat([q_rope, q_abs], -1), kv, block_table, seq_lens, sm_scale=self.sm_scale,
                               splits=getattr(self, "attn_splits", 1) or 1)
        return torch.bmm(o_lat.transpose(0, 1), wv_t).transpose(0, 1).reshape(t, hq * vd)

    def _mla_heads(self, h, layer):
        """Per-head (query, key, value) in the padded 256-wide layout: ``[T, 3 * Hq, 256]`` bf16, rows q | k | v."""
        cfg, m = self.cfg, layer.mla
        nope, rope, vd, hq = cfg.qk_nope_head_dim, cfg.qk_rope_head_dim, cfg.v_head_dim, self.hq
        t = h.shape[0]
        xq, xs = self._norm_quant(h, layer.attn_norm)
        if m.q_a is not None:
            q = m.q_b(*self._norm_quant(m.q_a(xq, xs), m.q_a_norm))
        else:
            q = m.q_b(xq, xs)
        ckv = m.kv_a(xq, xs)  # [T, kv_lora + rope]
        latent = ckv[:, : cfg.kv_lora_rank].contiguous()
        kvb = m.kv_b(*self._norm_quant(latent, m.kv_a_norm)).view(t, hq, nope + vd)
        q = q.view(t, hq, nope + rope)
        out = torch.zeros((t, 3 * hq, PADDED_HEAD), dtype=torch.bfloat16, device=h.device)
        out[:, :hq, :rope] = q[:, :, nope:]
        out[:, :hq, rope : rope + nope] = q[:, :, :nope]
        out[:, hq : 2 * hq, :rope] = ckv[:, None, cfg.kv_lora_rank :]  # one rotary key part shared by all heads
        out[:, hq : 2 * hq, rope : rope + nope] = kvb[:, :, :nope]
        out[:, 2 * hq :, :vd] = kvb[:, :, nope:]
        return out

    def _mla_attention(self, h, layer, kv, step: StepBuffers, prefill: bool):
        """Attention output in the shape ``o_proj`` consumes: ``[T, Hq * v_head_dim]``."""
        t = h.shape[0]
        qkv = self._mla_heads(h, layer).view(t, 3 * self.hq * PADDED_HEAD)
        o = self._attention(qkv, kv, step, prefill).view(t, self.hq, PADDED_HEAD)
        return o[:, :, : self.cfg.v_head_dim].reshape(t, self.hq * self.cfg.v_head_dim)

    def _block(self, h, layer, kv, step: StepBuffers, prefill: bool):
        if getattr(layer, "mla", None) is None:
            return super()._block(h, layer, kv, step, prefill)
        attn = (self._mla_absorbed if self.cfg.absorbed else self._mla_attention)(h, layer, kv, step, prefill)
        h = self._row_parallel(layer.o_proj, *self._in_plain(attn, layer.o_proj), h=h)
        return self._ffn(h, layer)


def random_mla_weights(cfg: MlaConfig, device, seed: int = 0, std: float = 0.02, expert_chunk: int = 32) -> MoeWeights:
    """N(0, std) weights in block FP8, drawn layer by layer on ``device`` (routed experts one chunk at a time)."""
    from .hybrid import _quant_stack
    dev = torch.device(device)
    gen = torch.Generator(device=dev)
    gen.manual_seed(seed)
    h, hq = cfg.hidden_size, cfg.num_heads
    nope, rope, vd = cfg.qk_nope_head_dim, cfg.qk_rope_head_dim, cfg.v_head_dim
    e, mi, si = cfg.num_experts, cfg.moe_intermediate, cfg.shared_intermediate

    def rnd(*shape, scale=std):
        return torch.randn(shape, generator=gen, device=dev, dtype=torch.float32).mul_(scale).to(torch.bfloat16)

    def ones(n):
        return torch.ones(n, dtype=torch.bfloat16, device=dev)

    def lin(n, k):
        return Fp8Linear.from_float(rnd(n, k))

    def experts(n, k):
        qs, ss = zip(*[_quant_stack(rnd(min(expert_chunk, e - lo), n, k)) for lo in range(0, e, expert_chunk)])
        return torch.cat(qs), torch.cat(ss)

    layers = []
    for i in range(cfg.num_layers):
        q_in = cfg.q_lora_rank or h
        mla = MlaWeights(lin(cfg.q_lora_rank, h) if cfg.q_lora_rank else None, ones(cfg.q_lora_rank) if cfg.q_lora_rank else None,
                         lin(hq * (nope + rope), q_in), lin(cfg.kv_lora_rank + rope, h), ones(cfg.kv_lora_rank),
                         lin(hq * (nope + vd), cfg.kv_lora_rank))
        layer = MlaLayer(attn_norm=ones(h), qkv=None, o_proj=lin(h, hq * vd), mlp_norm=ones(h), gate_up=None, down=None, mla=mla)
        if i < cfg.first_dense_layers:
            layer.gate_up, layer.down = lin(2 * cfg.intermediate_size, h), lin(h, cfg.intermediate_size)
        else:
            gu_q, gu_s = experts(2 * mi, h)
            dn_q, dn_s = experts(h, mi)
            bias = torch.randn(e, generator=gen, device=dev, dtype=torch.float32) * 0.01 if cfg.router == "sigmoid" else None
            layer.moe = MoeFfn(router=rnd(e, h), router_bias=bias, gate_up=gu_q, gate_up_scale=gu_s, down=dn_q, down_scale=dn_s)
            if si:
                layer.moe.shared_gate_up, layer.moe.shared_down = lin(2 * si, h), lin(h, si)
        layers.append(layer)
    return MoeWeights(rnd(cfg.vocab_size, h), layers, ones(h), lin(cfg.vocab_size, h), 0, 1)


def mla_weights_from_tensors(cfg: MlaConfig, tensors, device) -> MoeWeights:
    """Weights from checkpoint tensors under canonical names: the generic loader builds embeddings, norms, feed-forward
    blocks and ``o_proj`` (query / key / value of the plain attention do not exist in such a checkpoint and get zero
    stand-ins that are dropped again); the latent-attention projections are read here.  HF's rotary layout of the
    rope parts (interleaved pairs) is converted to the rotate-half layout this runtime uses."""
    import numpy as np
    from .moe_decoder import _to_float
    dev = torch.device(device)
    nope, rope, vd, hq = cfg.qk_nope_head_dim, cfg.qk_rope_head_dim, cfg.v_head_dim, cfg.num_heads

    class _View(dict):
        def __missing__(self, name):
            return tensors[name]

        def __contains__(self, name):
            return dict.__contains__(self, name) or name in tensors

    view = _View()
    for i in range(cfg.num_layers):
        p = f"model.block.{i}.attention."
        for n, rows in (("query", hq), ("key", hq), ("value", hq)):
            view[p + n + ".weight"] = np.zeros((rows * 128, cfg.hidden_size), dtype=np.float32)
    plain_cfg = MoeDecoderConfig(**{k: getattr(cfg, k) for k in MoeDecoderConfig.__dataclass_fields__})
    plain_cfg.head_dim = 128  # only sizes the stand-ins; o_proj takes its true width (Hq * v) from the tensor itself
    base = MoeWeights.from_tensors(plain_cfg, view, dev)

    def get(name):
        return _to_float(tensors[name], dev)

    def deinterleave(w, heads, lead):
        """Rows of every head: ``lead`` untouched rows, then ``rope`` rows stored as pairs (0,1),(2,3).. -> halves."""
        w = w.reshape(heads, lead + rope, -1)
        r = w[:, lead:]
        r = torch.cat([r[:, 0::2], r[:, 1::2]], 1)
        return torch.cat([w[:, :lead], r], 1).reshape(heads * (lead + rope), -1)

    layers = []
    for i, layer in enumerate(base.layers):
        p = f"model.block.{i}.attention."
        q_a = q_a_norm = None
        if cfg.q_lora_rank:
            q_a = Fp8Linear.from_float(get(p + "query_a.weight"))
            q_a_norm = get(p + "query_a_norm.weight").to(torch.bfloat16)
        kv_a = get(p + "key_value_a.weight")
        kv_a = torch.cat([kv_a[: cfg.kv_lora_rank], deinterleave(kv_a[cfg.kv_lora_rank :], 1, 0)], 0)
        mla = MlaWeights(q_a, q_a_norm, Fp8Linear.from_float(deinterleave(get(p + "query_b.weight"), hq, nope)),
                         Fp8Linear.from_float(kv_a), get(p + "key_value_a_norm.weight").to(torch.bfloat16),
                         Fp8Linear.from_float(get(p + "key_value_b.source.weight")))
        ml = MlaLayer(**{k: getattr(layer, k) for k in layer.__dataclass_fields__}, mla=mla)
        ml.qkv = None
        layers.append(ml)
    return MoeWeights(base.embed, layers, base.final_norm, base.lm_head, 0, 1)


def init_mla_tensors(cfg: MlaConfig, seed: int = 0, std: float = 0.02) -> dict[str, torch.Tensor]:
    """Random weights of an MLA model under canonical names (tests, synthetic checkpoints), in HF's rotary layout."""
    from .moe_lm import MoeConfig, init_weights
    w = init_weights(MoeConfig(vocab_size=cfg.vocab_size, hidden_size=cfg.hidden_size, num_layers=cfg.num_layers,
                               num_heads=cfg.num_heads, num_kv_heads=cfg.num_heads, head_dim=cfg.v_head_dim,
                               num_experts=cfg.num_experts, top_k=cfg.top_k, moe_intermediate=cfg.moe_intermediate,
                               shared_intermediate=cfg.shared_intermediate), seed=seed, std=std)
    g = torch.Generator().manual_seed(seed + 17)
    rnd = lambda *shape: (torch.randn(shape, generator=g) * std).to(torch.bfloat16).float()
    h, hq = cfg.hidden_size, cfg.num_heads
    nope, rope, vd = cfg.qk_nope_head_dim, cfg.qk_rope_head_dim, cfg.v_head_dim
    for i in range(cfg.num_layers):
        p = f"model.block.{i}.attention."
        for n in ("query", "key", "value"):
            w.pop(p + n + ".weight", None)
        if cfg.q_lora_rank:
            w[p + "query_a.weight"] = rnd(cfg.q_lora_rank, h)
            w[p + "query_a_norm.weight"] = 1 + rnd(cfg.q_lora_rank)
        w[p + "query_b.weight"] = rnd(hq * (nope + rope), cfg.q_lora_rank or h)
        w[p + "key_value_a.weight"] = rnd(cfg.kv_lora_rank + rope, h)
        w[p + "key_value_a_norm.weight"] = 1 + rnd(cfg.kv_lora_rank)
        w[p + "key_value_b.source.weight"] = rnd(hq * (nope + vd), cfg.kv_lora_rank)
        w[p + "output.weight"] = rnd(h, hq * vd)
    return w
