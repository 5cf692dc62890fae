"""Hybrid decoder in the style of Qwen3-Next / Qwen3.5: Gated-DeltaNet layers interleaved with gated full attention,
mixture-of-experts (or dense) feed-forward blocks.

* linear-attention layers: ``qkv | z | b | a`` come out of ONE FP8 GEMM (the four projections share the input, so
  their weights are stacked), causal conv + SiLU, the gated delta-rule recurrence with fused gated RMSNorm
  (:mod:`mfq_b200.ops.gdn`), then the row-parallel output projection.  State per sequence: ``[Hv, dk, dv]`` fp32 and a
  three-token conv history; it is addressed by the engine's batch row.
* full-attention layers (every ``full_attention_interval``-th): per-head RMSNorm of q and k, partial rotary embedding,
  FP8 paged KV, and an output gate ``sigmoid(gate) * attention`` whose projection is stacked behind q|k|v in the same
  GEMM and applied inside the quantization that feeds ``o_proj``.
* feed-forward: the routed-experts block of :class:`~mfq_b200.models.moe_decoder.MoeDecoderModel` (shared expert
  included) or the dense SwiGLU block.

Canonical tensor names follow the reference schema (``mfq/architectures/tensor_schema.py:559-593``):
``model.block.N.linear_attention.{qkv,gate,alpha,beta,conv,output,norm}.weight``, ``...linear_attention.{a,dt_bias}``,
``model.block.N.attention.{query_norm,key_norm}.weight``; the reference runs this family through
``cpp_runtime/backends/cuda/models/qwen35/linear_attention.h``.
"""

from __future__ import annotations

from dataclasses import dataclass

import numpy as np
import torch

from .. import ops
from ..ops import gdn
from ..ops import reference as ref
from ..utils.profiler import scope
from .llama import Fp8Linear, LlamaLayer, StepBuffers
from .moe_decoder import MoeDecoderConfig, MoeDecoderModel, MoeFfn, MoeLayer, MoeWeights, _to_float


@dataclass
class HybridConfig(MoeDecoderConfig):
    full_attention_interval: int = 4  # layers 3, 7, 11 ... are full attention, the rest linear attention
    linear_k_heads: int = 16
    linear_v_heads: int = 32
    linear_head_dim: int = 128
    partial_rotary: float = 0.25
    qk_norm: bool = True
    attn_output_gate: bool = True
    name: str = "hybrid-gdn-fp8"

    def is_linear(self, layer: int) -> bool:
        return (layer + 1) % self.full_attention_interval != 0

    @property
    def conv_dim(self) -> int:
        return (2 * self.linear_k_heads + self.linear_v_heads) * self.linear_head_dim

    @classmethod
    def next_80b(cls) -> "HybridConfig":
        """Qwen3-Next-style 80B-total / 3B-active hybrid: 48 layers in a 3 linear : 1 full attention pattern, 512 routed
        experts (top 10) plus one shared expert per layer, 256-wide attention heads."""
        return cls(vocab_size=151936, hidden_size=2048, intermediate_size=5120, num_layers=48, num_heads=16, num_kv_heads=2,
                   head_dim=256, rope_theta=1e7, rms_eps=1e-6, num_experts=512, top_k=10, moe_intermediate=512,
                   shared_intermediate=512, full_attention_interval=4, linear_k_heads=16, linear_v_heads=32,
                   linear_head_dim=128, name="hybrid-next-80b-fp8")

    @classmethod
    def tiny(cls) -> "HybridConfig":
        return cls(vocab_size=1024, hidden_size=256, intermediate_size=512, num_layers=4, num_heads=4, num_kv_heads=2,
                   head_dim=128, rope_theta=1e6, rms_eps=1e-6, num_experts=8, top_k=2, moe_intermediate=128,
                   shared_intermediate=128, full_attention_interval=2, linear_k_heads=2, linear_v_heads=4,
                   linear_head_dim=128, name="tiny-hybrid-fp8")


@dataclass
class GdnWeights:
    in_proj: Fp8Linear  # rows: q | k | v | z | b | a
    conv_w: torch.Tensor  # [C, 4] fp32
    A_log: torch.Tensor  # [Hv] fp32
    dt_bias: torch.Tensor  # [Hv] fp32
    norm_w: torch.Tensor  # [dv] fp32
    out_proj: Fp8Linear  # [H, Hv*dv]
    k_heads: int
    v_heads: int


@dataclass
class HybridLayer(MoeLayer):
    gdn: GdnWeights | None = None
    q_norm: torch.Tensor | None = None  # [D] fp32
    k_norm: torch.Tensor | None = None
    gated: bool = False  # qkv rows are followed by the output-gate projection


class GdnState:
    """Recurrent state of the linear-attention layers for ``slots`` sequences (slot = engine batch row)."""

    def __init__(self, cfg: HybridConfig, slots: int, device, tp: int = 1) -> None:
        hv, d = cfg.linear_v_heads // tp, cfg.linear_head_dim
        c = cfg.conv_dim // tp
        n = sum(cfg.is_linear(i) for i in range(cfg.num_layers))
        self.index = {i: j for j, i in enumerate(i for i in range(cfg.num_layers) if cfg.is_linear(i))}
        self.conv = torch.zeros((n, slots, 3, c), dtype=torch.float32, device=device)
        self.state = torch.zeros((n, slots, hv, d, d), dtype=torch.float32, device=device)

        self._ckpt: dict[tuple[int, int], tuple[torch.Tensor, torch.Tensor]] = {}

    def reset(self, slot: int) -> None:
        self.conv[:, slot].zero_()
        self.state[:, slot].zero_()

    def checkpoints(self, rows: int, window: int):
        """Per-layer verify-window checkpoints ``(conv [n, rows, L, 3, C], state [n, rows, L, Hv, d, d])`` (allocated once
        per geometry; 2 MB per layer, row and window position at d = 128, Hv = 32)."""
        key = (rows, window)
        if key not in self._ckpt:
            n, _, _, c = self.conv.shape
            self._ckpt[key] = (torch.zeros((n, rows, window, 3, c), dtype=torch.float32, device=self.conv.device),
                               torch.zeros((n, rows, window) + tuple(self.state.shape[2:]), dtype=torch.float32, device=self.conv.device))
        return self._ckpt[key]

    def commit(self, rows: int, window: int, slots: torch.Tensor, keep: torch.Tensor) -> None:
        """After a verify window: every layer adopts the checkpoint of window position ``keep[b]`` for row ``b``."""
        conv_ck, state_ck = self.checkpoints(rows, window)
        for j in range(self.conv.shape[0]):
            gdn.select(state_ck[j], conv_ck[j], self.state[j], self.conv[j], slots, keep)

    def layer(self, i: int):
        j = self.index[i]
        return self.conv[j], self.state[j]


def _tensor_bytes(obj, seen=None) -> int:
    """Bytes of every tensor reachable through dataclass fields, lists and tuples of ``obj``."""
    seen = set() if seen is None else seen
    if isinstance(obj, torch.Tensor):
        if obj.data_ptr() in seen:
            return 0
        seen.add(obj.data_ptr())
        return obj.numel() * obj.element_size()
    if isinstance(obj, (list, tuple)):
        return sum(_tensor_bytes(o, seen) for o in obj)
    if hasattr(obj, "__dataclass_fields__"):
        return sum(_tensor_bytes(getattr(obj, f), seen) for f in obj.__dataclass_fields__)
    if hasattr(obj, "__dict__") and not isinstance(obj, type):
        return sum(_tensor_bytes(v, seen) for v in vars(obj).values() if isinstance(v, (torch.Tensor, list, tuple)) or hasattr(v, "__dataclass_fields__"))
    return 0


class HybridWeights(MoeWeights):
    def nbytes(self) -> int:
        return _tensor_bytes(self)

    @classmethod
    def from_tensors(cls, cfg: HybridConfig, tensors, device, tp_rank: int = 0, tp_size: int = 1) -> "HybridWeights":
        """Rank-local FP8 weights from canonical checkpoint tensors.  Linear-attention heads, like attention heads,
        are split over the ranks; their stacked input projection keeps the q | k | v | z | b | a row order per rank."""
        dev = torch.device(device)
        w = tp_size
        base = super().from_tensors(cfg, _with_placeholders(cfg, tensors), dev, tp_rank, tp_size)
        d = cfg.linear_head_dim
        hk, hv = cfg.linear_k_heads, cfg.linear_v_heads

        def get(name):
            return _to_float(tensors[name], dev)

        def rows(x, parts):
            return x.reshape(w, parts // w, *x.shape[1:])[tp_rank] if w > 1 else x

        layers = []
        for i, layer in enumerate(base.layers):
            p = f"model.block.{i}."
            hl = HybridLayer(**{k: getattr(layer, k) for k in layer.__dataclass_fields__})
            if cfg.is_linear(i):
                q = p + "linear_attention."
                qkv = get(q + "qkv.weight")  # [2*hk*d + hv*d, H] in q | k | v order
                wq, wk, wv = qkv[: hk * d], qkv[hk * d : 2 * hk * d], qkv[2 * hk * d :]
                stacked = torch.cat([rows(wq, hk * d), rows(wk, hk * d), rows(wv, hv * d), rows(get(q + "gate.weight"), hv * d),
                                     rows(get(q + "beta.weight"), hv), rows(get(q + "alpha.weight"), hv)], 0)
                conv = get(q + "conv.weight").reshape(-1, 4)  # [C, 4] (a [C, 1, 4] depthwise kernel flattens to this)
                conv = torch.cat([rows(conv[: hk * d], hk * d), rows(conv[hk * d : 2 * hk * d], hk * d), rows(conv[2 * hk * d :], hv * d)], 0)
                out_w = get(q + "output.weight")
                if w > 1:
                    out_w = out_w.reshape(out_w.shape[0], w, hv * d // w)[:, tp_rank].contiguous()
                hl.gdn = GdnWeights(Fp8Linear.from_float(stacked), conv.contiguous(), rows(get(q + "a"), hv).contiguous(),
                                    rows(get(q + "dt_bias"), hv).contiguous(), get(q + "norm.weight").contiguous(),
                                    Fp8Linear.from_float(out_w), hk // w, hv // w)
                hl.qkv = hl.o_proj = None
            else:
                a = p + "attention."
                if cfg.qk_norm:
                    hl.q_norm, hl.k_norm = get(a + "query_norm.weight").contiguous(), get(a + "key_norm.weight").contiguous()
                if cfg.attn_output_gate:
                    gate = rows(get(a + "gate.weight"), cfg.num_heads * cfg.head_dim)
                    hl.qkv = Fp8Linear.from_float(torch.cat([hl.qkv.dequant().to(dev), gate], 0))
                    hl.gated = True
            layers.append(hl)
        return cls(base.embed, layers, base.final_norm, base.lm_head, tp_rank, tp_size)


def _quant_stack(w: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """``[E, N, K]`` float -> (E4M3 ``[E, N, K]``, fp32 scales ``[E, N/128, K/128]``), N and K multiples of 128."""
    e, n, k = w.shape
    tiles = w.float().reshape(e, n // 128, 128, k // 128, 128)
    scale = (tiles.abs().amax(dim=(2, 4)) / 448.0).clamp_min(1e-12)
    q = (tiles / scale[:, :, None, :, None]).clamp(-448.0, 448.0).to(torch.float8_e4m3fn)
    return q.reshape(e, n, k).contiguous(), scale.contiguous()


def random_hybrid_weights(cfg: HybridConfig, device, seed: int = 0, std: float = 0.02, mtp: bool = False,
                          expert_chunk: int = 64, tp_rank: int = 0, tp_size: int = 1, expert_format: str = "fp8") -> HybridWeights:
    """N(0, std) weights drawn and quantized to block FP8 on ``device``, layer by layer.  Only one chunk of
    ``expert_chunk`` experts exists in float at a time, so the 80B configuration builds inside its FP8 footprint.
    Under tensor / expert parallelism every rank draws the (small) dense matrices in full from the common stream and keeps
    its slice, and draws only its own experts, each chunk from a generator seeded by the chunk's global position: all
    ranks hold shards of one and the same model, whatever ``tp_size`` is.

    ``expert_format="packed"``: the routed experts are random payloads in the packed run-time layout instead
    (``ops.packed.PackedExperts.synthetic``): every (expert, projection) draws its family from a seeded allocation
    over NINT 2 / 3 / 4 / 5 bit and MXFP4 averaging about 3.4 bits per weight in HBM (2.9 code bits), and stays packed."""
    from .llama import MtpHead, kv_head_rows
    dev = torch.device(device)
    gen = torch.Generator(device=dev)
    gen.manual_seed(seed)
    egen = torch.Generator(device=dev)
    w, r = tp_size, tp_rank
    h, d, hq, hkv = cfg.hidden_size, cfg.head_dim, cfg.num_heads, cfg.num_kv_heads
    ld, lk, lv = cfg.linear_head_dim, cfg.linear_k_heads, cfg.linear_v_heads
    e, mi, si = cfg.num_experts, cfg.moe_intermediate, cfg.shared_intermediate
    if e % w or hq % w or lk % w or lv % w or cfg.vocab_size % w:
        raise ValueError(f"heads / experts / vocabulary of {cfg.name} do not split over {w} ranks")
    e_per = e // w
    chunk = min(expert_chunk, e_per)
    while e_per % chunk:
        chunk -= 1
    counter = [0]  # global position of the next expert chunk: the same sequence on every rank

    def rnd(*shape, scale=std):
        return torch.randn(shape, generator=gen, device=dev, dtype=torch.float32).mul_(scale).to(torch.bfloat16)

    def ones(n):
        return torch.ones(n, dtype=torch.bfloat16, device=dev)

    def rows(x, parts):  # this rank's share of `parts` leading rows
        return x.reshape(w, parts // w, *x.shape[1:])[r] if w > 1 else x

    def cols(x, parts):
        return x.reshape(x.shape[0], w, parts // w)[:, r].contiguous() if w > 1 else x

    def experts(n, k):
        qs, ss = [], []
        for lo in range(0, e, chunk):
            mine = r * e_per <= lo < (r + 1) * e_per
            if mine:
                egen.manual_seed(seed * 1_000_003 + 7919 * counter[0] + 1)
                x = torch.randn((chunk, n, k), generator=egen, device=dev, dtype=torch.float32).mul_(std).to(torch.bfloat16)
                q, s_ = _quant_stack(x)
                qs.append(q)
                ss.append(s_)
            counter[0] += 1
        return torch.cat(qs), torch.cat(ss)

    layer_no = [0]

    def packed_experts(n, k, salt):
        from ..ops import packed as packed_ops
        # seeded allocation per (layer, expert, projection): 40 % NINT2, 35 % NINT3, 15 % NINT4, 5 % NINT5, 5 % MXFP4
        # (2.9 code bits on average; with group codes and anchors about 3.4 bits per weight in HBM)
        rng = np.random.default_rng(seed * 1_000_003 + 101 * layer_no[0] + salt)
        alloc = rng.choice([2, 3, 4, 5, 16], size=e, p=[0.4, 0.35, 0.15, 0.05, 0.05])
        return packed_ops.PackedExperts.synthetic(e_per, n, k, alloc[r * e_per : (r + 1) * e_per], dev, gs=32,
                                                  seed=seed * 7919 + 13 * layer_no[0] + salt, std=std)

    def moe():
        layer_no[0] += 1
        if expert_format == "packed":
            ffn = MoeFfn(router=rnd(e, h), router_bias=None, gate_up=None, gate_up_scale=None, down=None, down_scale=None,
                         e_lo=r * e_per, packed_gate_up=packed_experts(2 * mi, h, 1), packed_down=packed_experts(h, mi, 2))
        else:
            gu_q, gu_s = experts(2 * mi, h)
            dn_q, dn_s = experts(h, mi)
            ffn = MoeFfn(router=rnd(e, h), router_bias=None, gate_up=gu_q, gate_up_scale=gu_s, down=dn_q, down_scale=dn_s,
                         e_lo=r * e_per)
        if si:
            sg, su, sd = rnd(si, h), rnd(si, h), rnd(h, si)
            if w > 1 and (si // w) % 128 == 0:
                sg, su, sd = rows(sg, si), rows(su, si), cols(sd, si)
            else:
                ffn.shared_replicated = w > 1
            ffn.shared_gate_up = Fp8Linear.from_float(torch.cat([sg, su], 0))
            ffn.shared_down = Fp8Linear.from_float(sd)
        return ffn

    def attention(gated: bool):
        wq, wk, wv = rnd(hq * d, h), rnd(hkv * d, h), rnd(hkv * d, h)
        parts = [rows(wq, hq * d), kv_head_rows(wk, hkv, d, r, w), kv_head_rows(wv, hkv, d, r, w)]
        if gated:
            parts.append(rows(rnd(hq * d, h), hq * d))
        return Fp8Linear.from_float(torch.cat(parts, 0)), Fp8Linear.from_float(cols(rnd(h, hq * d), hq * d))

    layers = []
    for i in range(cfg.num_layers):
        layer = HybridLayer(attn_norm=ones(h), qkv=None, o_proj=None, mlp_norm=ones(h), gate_up=None, down=None, moe=moe())
        if cfg.is_linear(i):
            stacked = torch.cat([rows(rnd(lk * ld, h), lk * ld), rows(rnd(lk * ld, h), lk * ld), rows(rnd(lv * ld, h), lv * ld),
                                 rows(rnd(lv * ld, h), lv * ld), rows(rnd(lv, h), lv), rows(rnd(lv, h), lv)], 0)  # q | k | v | z | b | a
            conv = rnd(cfg.conv_dim, 4, scale=0.3).float()
            conv = torch.cat([rows(conv[: lk * ld], lk * ld), rows(conv[lk * ld : 2 * lk * ld], lk * ld), rows(conv[2 * lk * ld :], lv * ld)], 0)
            a_log = torch.zeros(lv, dtype=torch.float32, device=dev).uniform_(-2.0, 0.5, generator=gen)
            layer.gdn = GdnWeights(Fp8Linear.from_float(stacked), conv.contiguous(), rows(a_log, lv).contiguous(),
                                   rows(rnd(lv, scale=0.5).float(), lv).contiguous(), (1 + rnd(ld, scale=0.1).float()).contiguous(),
                                   Fp8Linear.from_float(cols(rnd(h, lv * ld), lv * ld)), lk // w, lv // w)
        else:
            layer.qkv, layer.o_proj = attention(cfg.attn_output_gate)
            layer.gated = bool(cfg.attn_output_gate)
            if cfg.qk_norm:
                layer.q_norm, layer.k_norm = (1 + rnd(d, scale=0.1).float()).contiguous(), (1 + rnd(d, scale=0.1).float()).contiguous()
        layers.append(layer)
    head = None
    if mtp:
        # the draft head: one dense-attention block with a routed FFN of its own, fed by eh_proj([embed; hidden])
        qkv, o_proj = attention(False)
        blk = HybridLayer(attn_norm=ones(h), qkv=qkv, o_proj=o_proj, mlp_norm=ones(h), gate_up=None, down=None, moe=moe())
        head = MtpHead(ones(h), ones(h), Fp8Linear.from_float(rnd(h, 2 * h)), blk)
    embed = rnd(cfg.vocab_size, h)
    lm_head = Fp8Linear.from_float(rows(rnd(cfg.vocab_size, h), cfg.vocab_size))
    return HybridWeights(embed, layers, ones(h), lm_head, r, w, head)


def _with_placeholders(cfg: HybridConfig, tensors):
    """The MoE loader reads q/k/v/o of every layer; linear-attention layers have none, so they get zero stand-ins
    (dropped again right after)."""
    class _View(dict):
        def __missing__(self, name):
            return tensors[name]

        def __contains__(self, name):
            return dict.__contains__(self, name) or name in tensors

    view = _View()
    import numpy as np
    h, d = cfg.hidden_size, cfg.head_dim
    for i in range(cfg.num_layers):
        if cfg.is_linear(i):
            p = f"model.block.{i}.attention."
            view[p + "query.weight"] = np.zeros((cfg.num_heads * d, h), dtype=np.float32)
            view[p + "key.weight"] = np.zeros((cfg.num_kv_heads * d, h), dtype=np.float32)
            view[p + "value.weight"] = np.zeros((cfg.num_kv_heads * d, h), dtype=np.float32)
            view[p + "output.weight"] = np.zeros((h, cfg.num_heads * d), dtype=np.float32)
    return view


def init_hybrid_weights(cfg: HybridConfig, seed: int = 0, std: float = 0.02) -> dict[str, torch.Tensor]:
    """Random bf16-representable weights of a hybrid model under canonical names (tests, synthetic benchmarks)."""
    from .moe_lm import MoeConfig, init_weights
    w = init_weights(MoeConfig(vocab_size=cfg.vocab_size, hidden_size=cfg.hidden_size, num_layers=cfg.num_layers,
                               num_heads=cfg.num_heads, num_kv_heads=cfg.num_kv_heads, head_dim=cfg.head_dim,
                               num_experts=cfg.num_experts, top_k=cfg.top_k, moe_intermediate=cfg.moe_intermediate,
                               shared_intermediate=cfg.shared_intermediate), seed=seed, std=std)
    g = torch.Generator().manual_seed(seed + 1)

    def rnd(*shape, scale=std):
        return (torch.randn(shape, generator=g) * scale).to(torch.bfloat16).float()

    h, d, hk, hv = cfg.hidden_size, cfg.linear_head_dim, cfg.linear_k_heads, cfg.linear_v_heads
    for i in range(cfg.num_layers):
        p = f"model.block.{i}."
        if cfg.is_linear(i):
            for name in ("query", "key", "value", "output"):
                del w[p + f"attention.{name}.weight"]
            q = p + "linear_attention."
            w[q + "qkv.weight"] = rnd(cfg.conv_dim, h)
            w[q + "gate.weight"] = rnd(hv * d, h)
            w[q + "alpha.weight"] = rnd(hv, h)
            w[q + "beta.weight"] = rnd(hv, h)
            w[q + "conv.weight"] = rnd(cfg.conv_dim, 1, 4, scale=0.5)
            w[q + "a"] = rnd(hv, scale=0.5)
            w[q + "dt_bias"] = rnd(hv, scale=0.5)
            w[q + "norm.weight"] = 1 + rnd(d, scale=0.1)
            w[q + "output.weight"] = rnd(h, hv * d)
        else:
            a = p + "attention."
            if cfg.qk_norm:
                w[a + "query_norm.weight"] = 1 + rnd(cfg.head_dim, scale=0.1)
                w[a + "key_norm.weight"] = 1 + rnd(cfg.head_dim, scale=0.1)
            if cfg.attn_output_gate:
                w[a + "gate.weight"] = rnd(cfg.num_heads * cfg.head_dim, h)
    return w


class HybridModel(MoeDecoderModel):
    """:class:`MoeDecoderModel` whose token mixer is, per layer, Gated DeltaNet or gated full attention."""

    def __init__(self, cfg: HybridConfig, weights, collective=None) -> None:
        super().__init__(cfg, weights, collective)
        self.state: GdnState | None = None
        self.rot = max(2, int(cfg.head_dim * cfg.partial_rotary) // 2 * 2)

    def make_state(self, slots: int) -> GdnState:
        self.state = GdnState(self.cfg, slots, self.w.embed.device, self.tp)
        return self.state

    # -- linear attention ---------------------------------------------------------------------------------------------
    def _gdn_mixer(self, h, layer: HybridLayer, li: int, step: StepBuffers):
        cfg, g = self.cfg, layer.gdn
        d = cfg.linear_head_dim
        xq, xs = self._norm_quant(h, layer.attn_norm)
        proj = g.in_proj(xq, xs)  # [T, C + Hv*d + 2*Hv]
        c = (2 * g.k_heads + g.v_heads) * d
        zw = g.v_heads * d
        mixed, z = proj[:, :c], proj[:, c : c + zw]
        b, a = proj[:, c + zw : c + zw + g.v_heads], proj[:, c + zw + g.v_heads : c + zw + 2 * g.v_heads]
        conv_state, state = self.state.layer(li)
        slots = step.state_slots
        L = h.shape[0] if step.cu_seqlens else step.q_len  # prefill: one sequence, the whole chunk; else the decode window
        if not h.is_cuda:
            mixed, z, a, b = (t.contiguous() for t in (mixed, z, a, b))
        conv_ck = state_ck = None
        if step.verify:
            rows = h.shape[0] // L
            conv_all, state_all = self.state.checkpoints(rows, L)
            j = self.state.index[li]
            conv_ck, state_ck = conv_all[j], state_all[j]
        qkv = gdn.conv(mixed, conv_state, g.conv_w, slots, L, conv_ckpt=conv_ck)
        y = gdn.recurrent(qkv, z, a, b, g.A_log, g.dt_bias, g.norm_w, state, slots, L, g.k_heads, g.v_heads, cfg.rms_eps,
                          ckpt=state_ck)
        yq, ys = self._quant(y)
        return self._row_parallel(g.out_proj, yq, ys, h=h)

    # -- gated attention ----------------------------------------------------------------------------------------------
    def _gated_attention(self, h, layer: HybridLayer, kv, step: StepBuffers, prefill: bool):
        cfg = self.cfg
        d, t = cfg.head_dim, h.shape[0]
        xq, xs = self._norm_quant(h, layer.attn_norm)
        qkv = layer.qkv(xq, xs)  # [T, (Hq + 2Hk) * D (+ Hq * D gate)]
        width = (self.hq + 2 * self.hk) * d
        gate = qkv[:, width:] if layer.gated else None
        if qkv.is_cuda:
            kd = vd = None
            if prefill:
                kd = torch.empty((t, self.hk, d), dtype=torch.bfloat16, device=qkv.device)
                vd = torch.empty_like(kd)
            q = ops.rope_kv_write(qkv, step.positions, step.slots, kv, n_q=self.hq, n_kv=self.hk, head_dim=d, theta=cfg.rope_theta,
                                  rot=self.rot, kd_out=kd, vd_out=vd, q_norm=layer.q_norm, k_norm=layer.k_norm,
                                  norm_eps=cfg.rms_eps, scaling=self.rope_scaling)
            if prefill:
                o = self._prefill_attention(q, kd, vd, kv, step)
            else:
                o = ops.paged_attn_decode(q, kv, step.block_table, step.seq_lens, sm_scale=self.sm_scale,
                                          splits=self.attn_splits, q_len=step.q_len)
            o = o.reshape(t, self.hq * d)
            aq, a_s = ops.kernels.gate_quant_rows(o, gate) if gate is not None else self._quant(o)
        else:
            q3 = qkv[:, :width].reshape(t, self.hq + 2 * self.hk, d)

            def headnorm(x, w):
                if w is None:
                    return x
                xf = x.float()
                return (xf * torch.rsqrt((xf * xf).mean(-1, keepdim=True) + cfg.rms_eps) * w).to(torch.bfloat16)
            q = ref.rope(headnorm(q3[:, : self.hq], layer.q_norm), step.positions, cfg.rope_theta, self.rot, self.rope_scaling)
            k = ref.rope(headnorm(q3[:, self.hq : self.hq + self.hk], layer.k_norm), step.positions, cfg.rope_theta, self.rot, self.rope_scaling)
            ref.write_kv(kv, k, q3[:, self.hq + self.hk :], step.slots)
            if prefill:
                o = self._prefill_attention(q, None, None, kv, step)
            else:
                o = ref.paged_attn_decode(q, kv, step.block_table, step.seq_lens, self.sm_scale, step.q_len)
            o = o.reshape(t, self.hq * d)
            if gate is not None:
                o = (o.float() * torch.sigmoid(gate.float())).to(torch.bfloat16)
            aq, a_s = self._quant(o)
        return self._row_parallel(layer.o_proj, aq, a_s, h=h)

    def _block(self, h, layer, kv, step: StepBuffers, prefill: bool):
        li = self._layer_index.get(id(layer))  # None: a block outside the stack (the MTP head's attention block)
        if getattr(layer, "gdn", None) is not None:
            with scope("mixer.gdn", h.device):
                h = self._gdn_mixer(h, layer, li, step)
        elif isinstance(layer, HybridLayer):
            with scope("mixer.gated_attn", h.device):
                h = self._gated_attention(h, layer, kv, step, prefill)
        else:
            return super()._block(h, layer, kv, step, prefill)
        return self._ffn(h, layer)

    def commit_verify(self, rows: int, window: int, slots: torch.Tensor, keep: torch.Tensor) -> None:
        self.state.commit(rows, window, slots, keep)

    def forward(self, step: StepBuffers, cache, **kw):
        if self.state is None:
            raise RuntimeError("call make_state(slots) before the first forward")
        self._layer_index = {id(l): i for i, l in enumerate(self.w.layers)}
        return super().forward(step, cache, **kw)

    def mtp_forward(self, step: StepBuffers, cache, hidden, **kw):
        self._layer_index = {id(l): i for i, l in enumerate(self.w.layers)}
        return super().mtp_forward(step, cache, hidden, **kw)
