"""Mixture-of-experts decoder on the GPU kernels: tensor-parallel attention, expert-parallel routed experts.

Layout under ``W`` ranks (one process per GPU): attention heads, the shared expert and dense FFN layers are
tensor-parallel exactly like :class:`~mfq_b200.models.llama.LlamaModel`; rank ``r`` additionally owns the routed
experts ``[r*E/W, (r+1)*E/W)``.  The residual stream is replicated, so every rank routes all tokens itself and
only gathers rows for its own experts; the weighted expert outputs (+ the shared expert's partial) of all ranks are
summed by the fused row all-reduce, which also adds the residual.  The reference broadcasts hidden states and
routes to every GPU and reduces partial outputs to a primary GPU (``cpp_runtime/backends/cuda/core/ffn.cpp:201-300``).

Weights of any checkpoint family (NINT, NVQ, MXFP4, FP8-128SQ, bf16; MFE pools for the experts) are transcoded at
load time to E4M3 with 128x128 fp32 block multipliers -- the one format the tensor-core GEMMs consume -- which at
B200 memory sizes (180 GB per GPU) holds even the 671B configuration at EP=8.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np
import torch

from .. import formats as F
from .. import ops
from ..ops import moe as moe_ops
from ..ops import reference as ref
from ..quantize.fp8_block import quantize_fp8_block_torch
from ..utils.profiler import scope
from .llama import kv_head_rows, Fp8Linear, LlamaConfig, LlamaLayer, LlamaModel, LlamaWeights


@dataclass
class MoeDecoderConfig(LlamaConfig):
    num_experts: int = 8
    top_k: int = 2
    moe_intermediate: int = 128
    shared_intermediate: int = 0
    router: str = "softmax"  # "softmax" | "sigmoid"
    norm_topk: bool = True
    routed_scale: float = 1.0
    n_group: int = 1
    topk_group: int = 1
    first_dense_layers: int = 0  # leading layers that use the dense FFN (DeepSeek-style)
    name: str = "moe-fp8"

    @classmethod
    def tiny(cls) -> "MoeDecoderConfig":
        return cls(vocab_size=1024, hidden_size=256, intermediate_size=512, num_layers=2, num_heads=4, num_kv_heads=2,
                   head_dim=128, rope_theta=1e6, rms_eps=1e-6, num_experts=8, top_k=2, moe_intermediate=128,
                   shared_intermediate=128, name="tiny-moe-fp8")


@dataclass
class MoeFfn:
    router: torch.Tensor  # [E, H] bf16
    router_bias: torch.Tensor | None
    gate_up: torch.Tensor  # [E_local, 2I, H] fp8
    gate_up_scale: torch.Tensor
    down: torch.Tensor  # [E_local, H, I] fp8
    down_scale: torch.Tensor
    shared_gate_up: Fp8Linear | None = None
    shared_down: Fp8Linear | None = None
    e_lo: int = 0
    residency: object | None = None  # ExpertResidency: experts live on the host, `gate_up`/`down` are its HBM arena
    shared_replicated: bool = False  # shared expert too narrow to shard on 128-wide blocks: every rank holds all of it
    # routed experts kept in their packed checkpoint codes (ops.packed.PackedExperts); gate_up / down are then unused
    packed_gate_up: object | None = None
    packed_down: object | None = None


@dataclass
class MoeLayer(LlamaLayer):
    moe: MoeFfn | None = None


def _stack_fp8(mats: list[torch.Tensor]) -> tuple[torch.Tensor, torch.Tensor]:
    qs, ss = zip(*[quantize_fp8_block_torch(m) for m in mats])
    return torch.stack(qs).contiguous(), torch.stack(ss).contiguous()


def _to_float(t, device) -> torch.Tensor:
    """Any checkpoint tensor object -> float32 torch tensor on ``device`` (decode on the host, upload)."""
    return torch.from_numpy(np.ascontiguousarray(F.dequantize(t))).to(device=device, dtype=torch.float32)


class MoeWeights(LlamaWeights):
    @classmethod
    def from_tensors(cls, cfg: MoeDecoderConfig, tensors, device, tp_rank: int = 0, tp_size: int = 1,
                     expert_slots: int | None = None, native_4bit: bool = False, lp_rank: int = 0, lp_size: int = 1,
                     layer_split=None, packed_experts: bool = False) -> "MoeWeights":
        """Build rank-local FP8 weights from checkpoint tensors under canonical names (a dict or an ``MfqStore``).
        ``expert_slots`` < experts per rank keeps the routed experts in (pinned) host memory behind an HBM arena of
        that many slots (:class:`~mfq_b200.engine.expert_residency.ExpertResidency`); such a model decodes eagerly.
        ``native_4bit`` (single GPU): attention and dense-FFN projections stored as NINT (<= 4 code bits) or MXFP4 keep
        their 4-bit codes and run through the in-pipeline-decode GEMM instead of being transcoded to FP8.
        ``packed_experts`` (GPU): routed experts stored as MFE pools of NINT (group size 24 / 32) or MXFP4 keep their
        packed codes in HBM and are decoded inside the expert kernels (``ops/packed.py``); a layer that holds an expert
        of another family falls back to the FP8 transcode."""
        dev = torch.device(device)
        h, d, w = cfg.hidden_size, cfg.head_dim, tp_size
        hq, hk = cfg.num_heads, cfg.num_kv_heads

        def get(name):
            return _to_float(tensors[name], dev)

        def rows(x, parts):
            return x.reshape(w, parts // w, -1)[tp_rank] if w > 1 else x

        def cols(x, parts):
            return x.reshape(x.shape[0], w, parts // w)[:, tp_rank].contiguous() if w > 1 else x

        def norm(name):
            return get(name).to(torch.bfloat16)

        def fp8_direct(names):
            """Checkpoint tensors that already are E4M3 + 128x128 fp32 multipliers (a checkpoint in the native layout)
            are adopted as they are -- stacked along the rows when every part holds whole 128-row blocks -- instead
            of being decoded to float and quantized again.  Single rank only (shards cut through the blocks)."""
            if w != 1:
                return None
            from ..formats.fp8sq import Fp8SqTensor
            parts = [tensors[n] for n in names]
            if not all(isinstance(p, Fp8SqTensor) and p.dtype == "FP8-128SQ" and p.scale_dtype == "F32" and p.row_q_bits is None
                       and tuple(p.block_shape) == (128, 128) and p.shape[1] % 128 == 0 for p in parts):
                return None
            if len(parts) > 1 and any(p.shape[0] % 128 for p in parts[:-1]):
                return None
            q = torch.from_numpy(np.concatenate([np.asarray(p.codes, dtype=np.uint8) for p in parts], 0)).to(dev).view(torch.float8_e4m3fn)
            sc = torch.from_numpy(np.concatenate([np.asarray(p.scales, dtype=np.float32) for p in parts], 0)).to(dev)
            return Fp8Linear(q.contiguous(), sc.contiguous())

        def linear(names, float_builder):
            """4-bit native when every named tensor allows it, FP8 blocks adopted directly when the checkpoint stores
            them, else FP8 from the float matrix ``float_builder()``."""
            direct = fp8_direct(names)
            if direct is not None:
                return direct
            if native_4bit and w == 1:
                from ..models.llama import W4Linear
                from ..ops import w4 as w4ops
                parts = [w4ops.from_checkpoint_tensor(tensors[n]) for n in names]
                if all(p is not None for p in parts):
                    try:
                        return W4Linear(w4ops.concat_rows(parts).to(dev))
                    except ValueError:
                        pass
            return Fp8Linear.from_float(float_builder())

        e_per = cfg.num_experts // w
        e_lo = tp_rank * e_per
        def build_layer(p):
            qkv_names = [p + f"attention.{n}.weight" for n in ("query", "key", "value")]
            layer = MoeLayer(
                attn_norm=norm(p + "attention.norm.weight"),
                qkv=linear(qkv_names, lambda: torch.cat([rows(get(qkv_names[0]), hq * d), kv_head_rows(get(qkv_names[1]), hk, d, tp_rank, w),
                                                         kv_head_rows(get(qkv_names[2]), hk, d, tp_rank, w)], 0)),
                o_proj=linear([p + "attention.output.weight"], lambda: cols(get(p + "attention.output.weight"), hq * d)),
                mlp_norm=norm(p + "mlp.norm.weight"), gate_up=None, down=None)
            packed_pair = None
            if (p + "mlp.router.weight") in tensors and packed_experts and dev.type == "cuda" and expert_slots is None:
                from ..ops import packed as packed_ops
                mine = range(e_lo, e_lo + e_per)
                pgu = packed_ops.pack_moe_projection([tensors[p + "mlp.experts.gate.weight"], tensors[p + "mlp.experts.up.weight"]], mine, dev)
                pdn = packed_ops.pack_moe_projection([tensors[p + "mlp.experts.down.weight"]], mine, dev) if pgu is not None else None
                packed_pair = (pgu, pdn) if pdn is not None else None
            if packed_pair is not None:
                bias_name = p + "mlp.router.bias"
                ffn = MoeFfn(router=norm(p + "mlp.router.weight"), router_bias=get(bias_name) if bias_name in tensors else None,
                             gate_up=None, gate_up_scale=None, down=None, down_scale=None, e_lo=e_lo,
                             packed_gate_up=packed_pair[0], packed_down=packed_pair[1])
            elif (p + "mlp.router.weight") in tensors:
                gate = get(p + "mlp.experts.gate.weight")[e_lo : e_lo + e_per]
                up = get(p + "mlp.experts.up.weight")[e_lo : e_lo + e_per]
                down = get(p + "mlp.experts.down.weight")[e_lo : e_lo + e_per]
                gu_q, gu_s = _stack_fp8([torch.cat([gate[e], up[e]], 0) for e in range(e_per)])
                dn_q, dn_s = _stack_fp8([down[e] for e in range(e_per)])
                bias_name = p + "mlp.router.bias"
                ffn = MoeFfn(router=norm(p + "mlp.router.weight"),
                             router_bias=get(bias_name) if bias_name in tensors else None,
                             gate_up=gu_q, gate_up_scale=gu_s, down=dn_q, down_scale=dn_s, e_lo=e_lo)
            if (p + "mlp.router.weight") in tensors:
                if packed_pair is None and expert_slots is not None and expert_slots < e_per:
                    from ..engine.expert_residency import ExpertResidency
                    ffn.residency = ExpertResidency(gu_q.cpu(), gu_s.cpu(), dn_q.cpu(), dn_s.cpu(), expert_slots, dev)
                    arena = ffn.residency.arena
                    ffn.gate_up, ffn.gate_up_scale, ffn.down, ffn.down_scale = arena.gate_up, arena.gate_up_scale, arena.down, arena.down_scale
                if (p + "mlp.shared_expert.gate.weight") in tensors:
                    si = cfg.shared_intermediate
                    sg, su, sd = (get(p + f"mlp.shared_expert.{n}.weight") for n in ("gate", "up", "down"))
                    if w > 1 and (si // w) % 128 == 0:
                        sg, su, sd = rows(sg, si), rows(su, si), cols(sd, si)
                    else:
                        ffn.shared_replicated = w > 1
                    ffn.shared_gate_up = Fp8Linear.from_float(torch.cat([sg, su], 0))
                    ffn.shared_down = Fp8Linear.from_float(sd)
                layer.moe = ffn
            else:
                i_ = cfg.intermediate_size
                layer.gate_up = linear([p + "mlp.gate.weight", p + "mlp.up.weight"],
                                       lambda: torch.cat([rows(get(p + "mlp.gate.weight"), i_), rows(get(p + "mlp.up.weight"), i_)], 0))
                layer.down = linear([p + "mlp.down.weight"], lambda: cols(get(p + "mlp.down.weight"), i_))
            return layer

        lp_ranges = None
        if lp_size > 1:  # layer placement: only this rank's contiguous range is built (None keeps the global index)
            if tp_size != 1:
                raise ValueError("layer placement and tensor / expert parallelism are mutually exclusive")
            from ..parallel.layer_parallel import plan_layers
            lp_ranges = plan_layers(cfg.num_layers, lp_size, layer_split)
        mine = range(*lp_ranges[lp_rank]) if lp_ranges else range(cfg.num_layers)
        layers = [build_layer(f"model.block.{i}.") if i in mine else None for i in range(cfg.num_layers)]
        head = rows(get("model.output.weight"), cfg.vocab_size)
        weights = cls(get("model.token_embedding.weight").to(torch.bfloat16), layers, norm("model.output_norm.weight"),
                      Fp8Linear.from_float(head), tp_rank, tp_size)
        weights.lp_rank, weights.lp_size, weights.lp_ranges = lp_rank, lp_size, lp_ranges
        if "predictor.fusion.weight" in tensors and lp_ranges is None:  # multi-token-prediction head (one block; fusion = [embedding | hidden])
            from .llama import MtpHead
            out_norm = "predictor.output_norm.weight"
            weights.mtp = MtpHead(enorm=norm("predictor.embedding_norm.weight"), hnorm=norm("predictor.hidden_norm.weight"),
                                  eh_proj=Fp8Linear.from_float(get("predictor.fusion.weight")),
                                  layer=build_layer("predictor.block.0."),
                                  final_norm=norm(out_norm) if out_norm in tensors else None)
        return weights


class MoeDecoderModel(LlamaModel):
    """:class:`LlamaModel` whose FFN is a routed mixture of experts wherever the layer carries one."""

    expert_parallel = None  # an ExpertParallel: token-sharded dispatch / combine for wide batches (see below)
    ep_min_tokens = 0

    def enable_expert_all_to_all(self, group, max_tokens: int, min_tokens: int | None = None) -> None:
        """Route batches of at least ``min_tokens`` tokens (default 16 per rank) through the all-to-all: every rank
        dispatches ITS slice of the tokens to the ranks that own their experts (FP8 rows pushed into the owners'
        receive tables), runs its experts on what arrives and returns the weighted sums, instead of every rank gathering
        rows of ALL tokens for its experts and the partial outputs being all-reduced.  Collective: call on every rank.
        ``max_tokens``: the largest batch (tokens of the whole step) that will take this path."""
        from ..parallel.expert_parallel import ExpertParallel
        cfg = self.cfg
        per_rank = -(-max_tokens // self.tp)
        self.expert_parallel = ExpertParallel(group, self.w.embed.device, num_experts=cfg.num_experts, top_k=cfg.top_k,
                                              hidden=cfg.hidden_size, max_tokens=per_rank)
        self.ep_min_tokens = 16 * self.tp if min_tokens is None else min_tokens

    def residencies(self) -> list:
        """The expert-residency managers of this model's layers (empty when every expert lives in HBM)."""
        return [l.moe.residency for l in self.w.layers if getattr(l, "moe", None) is not None and l.moe.residency is not None]

    def forward(self, step, cache, **kw):
        for r in self.residencies():
            if r.optimistic:
                r.begin_step()  # inside a captured step this is a memset node: each replay starts its own histogram
        return super().forward(step, cache, **kw)

    def _ffn_all_to_all(self, h, ffn: MoeFfn, xq, xs, ids, wt):
        """Token-sharded expert layer: my slice of the rows goes through dispatch -> local experts -> combine, the
        finished slices are gathered back into the replicated residual stream.  A replicated shared expert runs on my
        slice only and rides along in the combine; a tensor-parallel one runs on all rows and its partial sums are
        reduced afterwards (by every rank: the collectives must be issued in the same order everywhere)."""
        t, w, r = h.shape[0], self.tp, self.w.tp_rank
        per = t // w
        lo, hi = r * per, (r + 1) * per
        ep = self.expert_parallel
        extra = partial = None
        if ffn.shared_gate_up is not None:
            if ffn.shared_replicated:
                extra = ffn.shared_down(*ops.silu_mul_quant(ffn.shared_gate_up(xq[lo:hi], xs[lo:hi])))
            else:
                partial = ffn.shared_down(*ops.silu_mul_quant(ffn.shared_gate_up(xq, xs)))
        mine = ep.moe_ffn(xq[lo:hi], xs[lo:hi], ids[lo:hi].contiguous(), wt[lo:hi].contiguous(), ffn.gate_up, ffn.gate_up_scale,
                          ffn.down, ffn.down_scale, base=h[lo:hi], extra=extra, cap=per)
        self.collective.allgather_rows(mine, out=h)
        if partial is not None:
            h = self.collective.allreduce_rows(partial, h)
        return h

    def _ffn(self, h, layer):
        ffn = getattr(layer, "moe", None)
        if ffn is None:
            return super()._ffn(h, layer)
        with scope("ffn.moe", h.device):
            return self._ffn_moe(h, layer, ffn)

    def _ffn_moe(self, h, layer, ffn: MoeFfn):
        cfg = self.cfg
        if not h.is_cuda:
            return self._ffn_reference(h, layer, ffn)
        xq, xs, y, _ = ops.rmsnorm_quant(h, layer.mlp_norm, cfg.rms_eps, want_y=True)
        ids, wt = moe_ops.router_topk(y, ffn.router, cfg.top_k, bias=ffn.router_bias, sigmoid=cfg.router == "sigmoid",
                                      norm_topk=cfg.norm_topk, scale=cfg.routed_scale, n_group=cfg.n_group,
                                      topk_group=cfg.topk_group)
        t = h.shape[0]
        ep = self.expert_parallel
        if (ep is not None and ffn.packed_gate_up is None and ffn.residency is None and self.tp > 1
                and t >= self.ep_min_tokens and t % self.tp == 0 and t // self.tp <= ep.cap_max):
            return self._ffn_all_to_all(h, ffn, xq, xs, ids, wt)
        shared = None
        if ffn.shared_gate_up is not None and not (ffn.shared_replicated and self.w.tp_rank != 0):
            sq, ss = ops.silu_mul_quant(ffn.shared_gate_up(xq, xs))
            shared = ffn.shared_down(sq, ss)  # this rank's partial of the shared expert (rank 0's whole, if replicated)
        if ffn.packed_gate_up is not None:
            # experts in their packed checkpoint codes: decoded in registers inside the expert products
            from ..ops import packed as packed_ops
            if self.tp == 1:
                return packed_ops.moe_ffn_packed(y, ids, wt, ffn.packed_gate_up, ffn.packed_down, e_lo=ffn.e_lo, base=h,
                                                 extra=shared, out=h)
            partial = packed_ops.moe_ffn_packed(y, ids, wt, ffn.packed_gate_up, ffn.packed_down, e_lo=ffn.e_lo, base=None,
                                                extra=shared)
            return self.collective.allreduce_rows(partial, h)
        if ffn.residency is not None:
            # host-tier experts: translate expert -> arena slot (uploading what is missing), in waves if needed
            local = ids - ffn.e_lo
            local = torch.where((local >= 0) & (local < ffn.residency.n), local, torch.full_like(local, -1))
            if ffn.residency.optimistic:
                arena = ffn.residency.arena  # one pass over what is resident; the engine settles misses after the step
                part = moe_ops.moe_ffn_fp8(xq, xs, ffn.residency.translate(local), wt, arena.gate_up, arena.gate_up_scale,
                                           arena.down, arena.down_scale, e_lo=0, base=None).float()
            else:
                part = ffn.residency.run(local, lambda ids_slot, arena: moe_ops.moe_ffn_fp8(
                    xq, xs, ids_slot, wt, arena.gate_up, arena.gate_up_scale, arena.down, arena.down_scale, e_lo=0, base=None).float())
            if part is None:  # no token of this step uses a local expert
                part = torch.zeros_like(h, dtype=torch.float32)
            out = h.float() + part + (shared.float() if shared is not None else 0)
            partial = out.to(torch.bfloat16)
            if self.tp == 1:
                h.copy_(partial)
                return h
            return self.collective.allreduce_rows((part + (shared.float() if shared is not None else 0)).to(torch.bfloat16), h)
        if self.tp == 1:
            return moe_ops.moe_ffn_fp8(xq, xs, ids, wt, ffn.gate_up, ffn.gate_up_scale, ffn.down, ffn.down_scale,
                                       e_lo=ffn.e_lo, base=h, extra=shared, out=h)
        partial = moe_ops.moe_ffn_fp8(xq, xs, ids, wt, ffn.gate_up, ffn.gate_up_scale, ffn.down, ffn.down_scale,
                                      e_lo=ffn.e_lo, base=None, extra=shared)
        return self.collective.allreduce_rows(partial, h)

    def _ffn_reference(self, h, layer, ffn: MoeFfn):
        """fp32 restatement of the GPU path (same FP8 rounding points); under TP/EP every rank adds its experts' partial."""
        cfg = self.cfg
        xq, xs, y, _ = ref.rmsnorm_quant(h, layer.mlp_norm, cfg.rms_eps)
        logits = y.float() @ ffn.router.float().T
        scores = torch.sigmoid(logits) if cfg.router == "sigmoid" else torch.softmax(logits, -1)
        sel = scores + (ffn.router_bias if ffn.router_bias is not None else 0)
        if cfg.n_group > 1:
            per = cfg.num_experts // cfg.n_group
            gs = sel.view(-1, cfg.n_group, per).topk(2, -1).values.sum(-1)
            keep = torch.zeros_like(gs, dtype=torch.bool).scatter_(1, gs.topk(cfg.topk_group, -1).indices, True)
            sel = sel.masked_fill(~keep.repeat_interleave(per, 1), float("-inf"))
        ids = sel.topk(cfg.top_k, -1).indices
        wt = scores.gather(1, ids)
        if cfg.norm_topk:
            wt = wt / wt.sum(-1, keepdim=True).clamp_min(1e-20)
        wt = wt * cfg.routed_scale
        out = torch.zeros_like(h, dtype=torch.float32)  # this rank's experts (+ its share of the shared expert)
        xd = xq.float() * xs[:, None]
        # with an expert arena the fp32 path reads the host tier directly: all experts are there, no slot bookkeeping
        e_gu, e_gus, e_dn, e_dns = ffn.residency.host if ffn.residency is not None else (ffn.gate_up, ffn.gate_up_scale, ffn.down, ffn.down_scale)
        for le in range(e_gu.shape[0]):
            tok, slot = (ids == ffn.e_lo + le).nonzero(as_tuple=True)
            if tok.numel() == 0:
                continue
            gu = (xd[tok] @ ref.dequant_block(e_gu[le], e_gus[le]).T).to(torch.bfloat16)
            hq, hs = ref.silu_mul_quant(gu)
            ye = ((hq.float() * hs[:, None]) @ ref.dequant_block(e_dn[le], e_dns[le]).T).to(torch.bfloat16)
            out.index_add_(0, tok, ye.float() * wt[tok, slot][:, None])
        if ffn.shared_gate_up is not None and not (ffn.shared_replicated and self.w.tp_rank != 0):
            sq, ss = ref.silu_mul_quant(ffn.shared_gate_up(xq, xs))
            out += ffn.shared_down(sq, ss).float()
        if self.tp > 1:
            return self.collective.allreduce_rows(out.to(torch.bfloat16), h)
        return (h.float() + out).to(torch.bfloat16)
