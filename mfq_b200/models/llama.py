"""Dense Llama-style decoder in block-scaled FP8 (weights E4M3 + 128x128 fp32 multipliers, FP8 paged KV).

One module, two execution paths with identical quantization semantics:

* ``device.type == "cuda"``: the hand-written kernels of :mod:`mfq_b200.ops` (tcgen05 FP8 GEMM with the
  residual add fused in its epilogue, fused RMSNorm+quant, RoPE+page write, paged decode attention);
* CPU: the fp32 restatements in :mod:`mfq_b200.ops.reference` (the oracle of the tests).

Projections are stored fused (``qkv``, ``gate_up``) and, under tensor parallelism, pre-sharded per rank:
column shards for ``qkv``/``gate_up`` (whole heads / whole 128-row blocks per rank), input shards for
``o_proj``/``down``, so each rank's shard keeps the 128x128 scale grid intact.  The canonical checkpoint names
(``model.block.N.attention.query.weight`` ...) follow the reference schema
(``mfq/architectures/tensor_schema.py:551-596``); axis rules follow ``ops/include/cuda_execution.h:179-197``.
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch

from .. import ops
from ..ops import reference as ref
from ..quantize.fp8_block import quantize_fp8_block_torch
from ..utils.profiler import scope
from .rope_scaling import YarnScaling

FP8 = torch.float8_e4m3fn


@dataclass
class LlamaConfig:
    vocab_size: int = 128256
    hidden_size: int = 4096
    intermediate_size: int = 14336
    num_layers: int = 32
    num_heads: int = 32
    num_kv_heads: int = 8
    head_dim: int = 128
    rope_theta: float = 5e5
    rms_eps: float = 1e-5
    max_position: int = 8192
    name: str = "llama-8b-fp8"
    rope_scaling: dict | None = None  # YaRN context extension: the fields of models.rope_scaling.YarnScaling

    @classmethod
    def llama_8b(cls) -> "LlamaConfig":
        return cls()

    @classmethod
    def tiny(cls) -> "LlamaConfig":
        return cls(vocab_size=1024, hidden_size=256, intermediate_size=512, num_layers=2, num_heads=4, num_kv_heads=2,
                   head_dim=128, rope_theta=1e4, name="llama-tiny-fp8")

    def param_count(self) -> int:
        h, i = self.hidden_size, self.intermediate_size
        per = h * (self.num_heads + 2 * self.num_kv_heads) * self.head_dim + self.num_heads * self.head_dim * h + 3 * h * i
        return self.num_layers * per + 2 * self.vocab_size * h


@dataclass
class Fp8Linear:
    """``[out, in]`` E4M3 codes + ``[ceil(out/128), in/128]`` fp32 multipliers."""

    q: torch.Tensor
    scale: torch.Tensor
    input_kind = "fp8"  # consumes per-row quantized E4M3 activations

    @classmethod
    def from_float(cls, w: torch.Tensor) -> "Fp8Linear":
        q, s = quantize_fp8_block_torch(w)
        return cls(q, s)

    def __call__(self, x_q: torch.Tensor, x_scale: torch.Tensor, residual: torch.Tensor | None = None, out=None):
        if x_q.is_cuda:
            return ops.fp8_gemm(x_q, x_scale, self.q, self.scale, residual=residual, out=out)
        return ref.fp8_gemm(x_q, x_scale, self.q, self.scale, residual=residual)

    def dequant(self) -> torch.Tensor:
        return ref.dequant_block(self.q, self.scale)


@dataclass
class W4Linear:
    """4-bit group-quantized weights decoded inside the GEMM pipeline (``ops/csrc/w4_gemm.cu``): the NINT-native
    path for code widths up to 4 bits.  Consumes bf16 activations."""

    w: "object"  # ops.w4.W4Weight
    input_kind = "bf16"

    @classmethod
    def from_float(cls, w: torch.Tensor, group_size: int = 32) -> "W4Linear":
        from ..ops import w4
        return cls(w4.quantize_torch(w, group_size))

    @classmethod
    def from_nint(cls, t, device) -> "W4Linear":
        from ..ops import w4
        return cls(w4.from_nint(t).to(device))

    def __call__(self, x: torch.Tensor, residual: torch.Tensor | None = None, out=None):
        from ..ops import w4
        return w4.w4_gemm(x, self.w, residual=residual, out=out)

    def dequant(self) -> torch.Tensor:
        from ..ops import w4
        return w4.dequantize(self.w)


@dataclass
class LlamaLayer:
    attn_norm: torch.Tensor
    qkv: Fp8Linear
    o_proj: Fp8Linear
    mlp_norm: torch.Tensor
    gate_up: Fp8Linear
    down: Fp8Linear


@dataclass
class MtpHead:
    """Multi-token-prediction module: ``z = eh_proj([rmsnorm(embed(next token)); rmsnorm(hidden)])`` followed by one
    decoder block with its own KV layer; the output norm and the LM head are the main model's unless it has its own
    norm (DeepSeek-V3 / Qwen3-Next style; reference: ``cpp_runtime/backends/cuda/engine/mtp.cpp``)."""

    enorm: torch.Tensor
    hnorm: torch.Tensor
    eh_proj: Fp8Linear  # [H, 2H], replicated under tensor parallelism
    layer: LlamaLayer
    final_norm: torch.Tensor | None = None


def kv_head_rows(w: torch.Tensor, kv_heads: int, head_dim: int, rank: int, world: int) -> torch.Tensor:
    """Rows of a K or V projection that rank ``rank`` of ``world`` keeps: ``kv_heads / world`` heads each while there are
    enough of them, else the single head that the rank's query heads share (that head is then replicated over
    ``world / kv_heads`` ranks, each of which caches it)."""
    if world == 1:
        return w
    if kv_heads >= world:
        if kv_heads % world:
            raise ValueError(f"{kv_heads} KV heads do not split over {world} ranks")
        per = kv_heads // world * head_dim
        return w[rank * per : (rank + 1) * per]
    if world % kv_heads:
        raise ValueError(f"{world} ranks do not split over {kv_heads} KV heads")
    head = rank // (world // kv_heads)
    return w[head * head_dim : (head + 1) * head_dim]


@dataclass
class LlamaWeights:
    embed: torch.Tensor  # [V, H] bf16
    layers: list[LlamaLayer]
    final_norm: torch.Tensor
    lm_head: Fp8Linear
    tp_rank: int = 0
    tp_size: int = 1
    mtp: MtpHead | None = None

    @classmethod
    def random_init(cls, cfg: LlamaConfig, device, seed: int = 0, std: float = 0.02, tp_rank: int = 0,
                    tp_size: int = 1, mtp: bool = False, weight_format: str = "fp8") -> "LlamaWeights":
        """N(0, std) weights, quantized layer by layer on ``device``.  Every rank draws the full matrix from the
        same seed and keeps its shard, so TP=n and TP=1 hold the same model."""
        dev = torch.device(device)
        gen = torch.Generator(device=dev)
        gen.manual_seed(seed)
        h, i, d = cfg.hidden_size, cfg.intermediate_size, cfg.head_dim
        hq, hk = cfg.num_heads, cfg.num_kv_heads

        def rnd(rows, cols):
            return torch.randn((rows, cols), generator=gen, device=dev, dtype=torch.float32).mul_(std).to(torch.bfloat16)

        lin = W4Linear.from_float if weight_format == "w4" else Fp8Linear.from_float  # block linears; the head stays FP8
        if weight_format == "w4" and tp_size > 1:
            raise ValueError("the 4-bit path is single-GPU for now")

        def rows_shard(w, parts):  # split output rows into tp_size equal shards, keep ours
            return w.reshape(tp_size, parts // tp_size, -1)[tp_rank] if tp_size > 1 else w

        layers = []
        for _ in range(cfg.num_layers + (1 if mtp else 0)):  # the last one becomes the MTP block
            wq, wk, wv = rnd(hq * d, h), rnd(hk * d, h), rnd(hk * d, h)
            wo = rnd(h, hq * d)
            wg, wu, wd = rnd(i, h), rnd(i, h), rnd(h, i)
            if tp_size > 1:
                wq = rows_shard(wq, hq * d)
                wk, wv = kv_head_rows(wk, hk, d, tp_rank, tp_size), kv_head_rows(wv, hk, d, tp_rank, tp_size)
                wg, wu = rows_shard(wg, i), rows_shard(wu, i)
                wo = wo.reshape(h, tp_size, hq * d // tp_size)[:, tp_rank].contiguous()
                wd = wd.reshape(h, tp_size, i // tp_size)[:, tp_rank].contiguous()
            layers.append(LlamaLayer(
                attn_norm=torch.ones(h, dtype=torch.bfloat16, device=dev),
                qkv=lin(torch.cat([wq, wk, wv], 0)),
                o_proj=lin(wo),
                mlp_norm=torch.ones(h, dtype=torch.bfloat16, device=dev),
                gate_up=lin(torch.cat([wg, wu], 0)),
                down=lin(wd),
            ))
            del wq, wk, wv, wo, wg, wu, wd
        embed = rnd(cfg.vocab_size, h)
        head = rnd(cfg.vocab_size, h)
        if tp_size > 1:
            head = rows_shard(head, cfg.vocab_size)
        head_module = None
        if mtp:
            ones = torch.ones(h, dtype=torch.bfloat16, device=dev)
            head_module = MtpHead(ones.clone(), ones.clone(), Fp8Linear.from_float(rnd(h, 2 * h)), layers.pop())
        return cls(embed, layers, torch.ones(h, dtype=torch.bfloat16, device=dev), Fp8Linear.from_float(head),
                   tp_rank, tp_size, head_module)

    def nbytes(self) -> int:
        total = self.embed.numel() * 2 + self.lm_head.q.numel()
        for l in self.layers:
            for lin in (l.qkv, l.o_proj, l.gate_up, l.down):
                total += lin.q.numel() + lin.scale.numel() * 4
        return total


@dataclass
class StepBuffers:
    """Device tensors describing one forward pass."""

    input_ids: torch.Tensor  # [T] int32
    positions: torch.Tensor  # [T] int32
    slots: torch.Tensor  # [T] int32 physical KV slot per token (-1 = do not write)
    # decode: one row per sequence
    block_table: torch.Tensor | None = None  # [B, max_pages] int32
    seq_lens: torch.Tensor | None = None  # [B] int32, length *after* this step's token
    # prefill: cumulative sequence boundaries (host list) of the packed chunk
    cu_seqlens: list[int] = field(default_factory=list)
    q_len: int = 1
    # models with recurrent state (linear attention): state slot of every row ([B] int32, -1 = leave the row alone)
    state_slots: torch.Tensor | None = None
    # MTP verify window: recurrent layers write per-token state checkpoints instead of committing their state;
    # the engine commits the checkpoint of the last accepted token afterwards
    verify: bool = False
    # chunked prefill / restored prefix: tokens of the sequence that are already in the KV pages (the chunk attends to
    # them too); the chunk must then be a single sequence and `block_table` its page-id row ([1, max_pages])
    past_len: int = 0


class LlamaModel:
    """Stateless forward over :class:`LlamaWeights`; KV state lives in a :class:`PagedKVCache`."""

    def __init__(self, cfg: LlamaConfig, weights: LlamaWeights, collective=None) -> None:
        self.cfg, self.w = cfg, weights
        self.tp = weights.tp_size
        self.collective = collective  # tensor-parallel reducer (None at TP=1)
        self.hq = cfg.num_heads // self.tp
        self.hk = max(1, cfg.num_kv_heads // self.tp)
        self.sm_scale = 1.0 / math.sqrt(cfg.head_dim)
        self.rope_scaling = YarnScaling.from_dict(getattr(cfg, "rope_scaling", None))
        if self.rope_scaling is not None:
            self.sm_scale *= self.rope_scaling.softmax_scale_factor
        self.attn_splits = 1
        self.attn_rot = None  # leading dims of a head that are rotated (None: all of them)

    # -- primitive dispatch -------------------------------------------------------------------------------------
    def _norm_quant(self, x, w):
        if x.is_cuda:
            q, s, _, _ = ops.rmsnorm_quant(x, w, self.cfg.rms_eps)
            return q, s
        q, s, _, _ = ref.rmsnorm_quant(x, w, self.cfg.rms_eps)
        return q, s

    def _quant(self, x):
        return ops.quant_rows(x) if x.is_cuda else ref.quant_rows(x)

    def _silu_quant(self, gu):
        return ops.silu_mul_quant(gu) if gu.is_cuda else ref.silu_mul_quant(gu)

    def _row_parallel(self, lin, *x_in, h):
        """Input-sharded projection + residual.  At TP>1 every rank adds its partial; rank 0 carries the residual."""
        if self.tp == 1:
            return lin(*x_in, residual=h, out=h if h.is_cuda else None)
        return self.collective.row_parallel_linear(lin, *x_in, h)

    # inputs of a linear in the form it consumes: (fp8 rows, multipliers) or (bf16,)
    def _in_norm(self, h, norm_w, lin):
        if lin.input_kind == "bf16":
            if h.is_cuda:
                return (ops.rmsnorm_quant(h, norm_w, self.cfg.rms_eps, want_q=False, want_y=True)[2],)
            return (ref.rmsnorm(h, norm_w, self.cfg.rms_eps),)
        return self._norm_quant(h, norm_w)

    def _in_plain(self, x, lin):
        return (x,) if lin.input_kind == "bf16" else self._quant(x)

    def _in_silu(self, gu, lin):
        if lin.input_kind == "bf16":
            if gu.is_cuda:
                return (ops.kernels.silu_mul(gu),)
            i = gu.shape[1] // 2
            return ((torch.nn.functional.silu(gu[:, :i].float()) * gu[:, i:].float()).to(torch.bfloat16),)
        return self._silu_quant(gu)

    # -- attention ----------------------------------------------------------------------------------------------
    def _attention(self, qkv, kv, step: StepBuffers, prefill: bool):
        cfg = self.cfg
        d = cfg.head_dim
        t = qkv.shape[0]
        kd = vd = None
        if qkv.is_cuda:
            if prefill:
                kd = torch.empty((t, self.hk, d), dtype=torch.bfloat16, device=qkv.device)
                vd = torch.empty_like(kd)
            q = ops.rope_kv_write(qkv, step.positions, step.slots, kv, n_q=self.hq, n_kv=self.hk, head_dim=d,
                                  theta=cfg.rope_theta, rot=self.attn_rot, kd_out=kd, vd_out=vd, scaling=self.rope_scaling)
        else:
            q3 = qkv.view(t, self.hq + 2 * self.hk, d)
            q = ref.rope(q3[:, : self.hq], step.positions, cfg.rope_theta, self.attn_rot, self.rope_scaling)
            k = ref.rope(q3[:, self.hq : self.hq + self.hk], step.positions, cfg.rope_theta, self.attn_rot, self.rope_scaling)
            ref.write_kv(kv, k, q3[:, self.hq + self.hk :], step.slots)
        if not prefill:
            if qkv.is_cuda:
                o = ops.paged_attn_decode(q, kv, step.block_table, step.seq_lens, sm_scale=self.sm_scale,
                                          splits=self.attn_splits, q_len=step.q_len)
            else:
                o = ref.paged_attn_decode(q, kv, step.block_table, step.seq_lens, self.sm_scale, step.q_len)
            return o.reshape(t, self.hq * d)
        return self._prefill_attention(q, kd, vd, kv, step).reshape(t, self.hq * d)

    def _prefill_attention(self, q, kd, vd, kv, step: StepBuffers):
        """Causal attention of a prefill chunk, ``[T, Hq, D]``.  Each sequence of a packed chunk attends to itself,
        through the same FP8 rounding of K/V that later decode steps read back from the pages (``kd`` / ``vd`` on the
        GPU); a chunk with ``past_len`` > 0 also attends to the sequence's cached past."""
        if step.past_len > 0:
            row = step.block_table[0]
            if q.is_cuda:
                kp, vp = ops.kernels.kv_gather_dequant(kv, row, step.past_len)
                return ops.kernels.attn_prefill_bf16(q, torch.cat([kp, kd], 0), torch.cat([vp, vd], 0), self.sm_scale)
            ps = kv.page_size
            past = torch.arange(step.past_len)
            kp, vp = ref.gather_slots(kv, row[(past // ps).long()] * ps + past % ps)
            kc, vc = ref.gather_slots(kv, step.slots)
            return ref.attention(q, torch.cat([kp, kc], 0), torch.cat([vp, vc], 0), self.sm_scale, causal_offset=step.past_len)
        if q.is_cuda:
            return ops.attn_prefill(q, kd, vd, step.cu_seqlens, self.sm_scale)
        outs = []
        for i in range(len(step.cu_seqlens) - 1):
            a, b = step.cu_seqlens[i], step.cu_seqlens[i + 1]
            kk, vv = ref.gather_slots(kv, step.slots[a:b])
            outs.append(ref.attention(q[a:b], kk, vv, self.sm_scale, causal_offset=0))
        return torch.cat(outs, 0)

    def _self_prepared(self, lin, rows: int) -> bool:
        """Whether ``lin`` takes bf16 rows and prepares its FP8 activations inside its own kernel: a few rows on one GPU
        (``ops.fp8_gemv_act``) -- four kernels less per layer in a single-stream decode step, same bits."""
        return (self.tp == 1 and isinstance(lin, Fp8Linear) and lin.q.is_cuda and lin.q.ndim == 2
                and ops.act_gemv_pays(rows, lin.q.shape[0], lin.q.shape[1]))

    # -- feed-forward -------------------------------------------------------------------------------------------
    def _ffn(self, h, layer):
        """Dense SwiGLU block: ``h + down(silu(gate(x)) * up(x))`` with ``x = rmsnorm(h)``."""
        rows = h.shape[0]
        with scope("ffn.gate_up", h.device):
            if self._self_prepared(layer.gate_up, rows):
                gu = ops.fp8_gemv_act(h, layer.gate_up.q, layer.gate_up.scale, ops.ACT_NORM, norm_w=layer.mlp_norm,
                                      eps=self.cfg.rms_eps)
            else:
                gu = layer.gate_up(*self._in_norm(h, layer.mlp_norm, layer.gate_up))
        with scope("ffn.down", h.device):
            if self._self_prepared(layer.down, rows) and gu.shape[1] == 2 * layer.down.q.shape[1]:
                return ops.fp8_gemv_act(gu, layer.down.q, layer.down.scale, ops.ACT_SWIGLU, residual=h, out=h)
            return self._row_parallel(layer.down, *self._in_silu(gu, layer.down), h=h)

    # -- forward ------------------------------------------------------------------------------------------------
    def _embed(self, ids):
        return ops.embed(ids, self.w.embed) if self.w.embed.is_cuda else self.w.embed[ids.long()].clone()

    def _block(self, h, layer, kv, step: StepBuffers, prefill: bool):
        rows = h.shape[0]
        with scope("attn.qkv", h.device):
            if self._self_prepared(layer.qkv, rows):
                qkv = ops.fp8_gemv_act(h, layer.qkv.q, layer.qkv.scale, ops.ACT_NORM, norm_w=layer.attn_norm, eps=self.cfg.rms_eps)
            else:
                qkv = layer.qkv(*self._in_norm(h, layer.attn_norm, layer.qkv))
        with scope("attn.core", h.device):
            attn = self._attention(qkv, kv, step, prefill)
        with scope("attn.o_proj", h.device):
            if self._self_prepared(layer.o_proj, rows) and attn.is_contiguous():
                h = ops.fp8_gemv_act(attn, layer.o_proj.q, layer.o_proj.scale, ops.ACT_PLAIN, residual=h, out=h)
            else:
                h = self._row_parallel(layer.o_proj, *self._in_plain(attn, layer.o_proj), h=h)
        return self._ffn(h, layer)

    def _head(self, h, norm, gather_logits: bool):
        with scope("head", h.device):
            xq, xs = self._norm_quant(h, norm)
            logits = self.w.lm_head(xq, xs)
            if self.tp > 1 and gather_logits:
                logits = self.collective.gather_columns(logits)
        return logits

    @property
    def local_layers(self) -> int:
        """Layers whose weights and KV pages this rank holds (all of them unless layers are placed across ranks)."""
        ranges = getattr(self.w, "lp_ranges", None)
        if not ranges:
            return len(self.w.layers)
        l0, l1 = ranges[self.w.lp_rank]
        return l1 - l0

    def _fused_tp(self, rows: int) -> bool:
        """Whether this pass takes the fused tensor-parallel pipeline: the plain dense block, FP8 linears, a collective
        that offers the fused reduce, and a row count within its buffers."""
        col = self.collective
        return (self.tp > 1 and type(self)._block is LlamaModel._block and type(self)._ffn is LlamaModel._ffn
                and hasattr(col, "row_parallel_fused") and getattr(col, "fused", True)
                and not getattr(self.w, "lp_ranges", None) and rows <= col.fused_rows(self.cfg.hidden_size)
                and all(l.qkv.input_kind == "fp8" for l in self.w.layers[:1]))

    def _run_layers_fused(self, h, step: StepBuffers, cache, prefill: bool):
        """Tensor-parallel layer stack with every all-reduce fused with the residual add, the FOLLOWING RMSNorm and
        its FP8 quantization (one kernel per row-parallel projection).  Returns the residual stream and the rows
        already normalised with the output norm and quantised: the LM head's input."""
        w, eps, col = self.w, self.cfg.rms_eps, self.collective
        x = self._norm_quant(h, w.layers[0].attn_norm)
        last = len(w.layers) - 1
        for li, layer in enumerate(w.layers):
            with scope("attn.qkv", h.device):
                qkv = layer.qkv(*x)
            with scope("attn.core", h.device):
                attn = self._attention(qkv, cache.layer(li), step, prefill)
            with scope("attn.o_proj", h.device):
                h, xq, xs = col.row_parallel_fused(layer.o_proj, *self._quant(attn), h, layer.mlp_norm, eps)
            with scope("ffn.gate_up", h.device):
                gu = layer.gate_up(xq, xs)
            with scope("ffn.down", h.device):
                nxt = w.layers[li + 1].attn_norm if li < last else w.final_norm
                h, xq, xs = col.row_parallel_fused(layer.down, *self._silu_quant(gu), h, nxt, eps)
            x = (xq, xs)
        return h, x

    def _run_layers(self, h, step: StepBuffers, cache, prefill: bool):
        w = self.w
        ranges = getattr(w, "lp_ranges", None)
        if not ranges:
            for li, layer in enumerate(w.layers):
                h = self._block(h, layer, cache.layer(li), step, prefill)
            return h
        # layer placement: stages run one after the other; the owner's result reaches every rank
        for stage, (l0, l1) in enumerate(ranges):
            if stage == w.lp_rank:
                for li in range(l0, l1):
                    h = self._block(h, w.layers[li], cache.layer(li - l0), step, prefill)
            h = self.collective.broadcast_rows(h, stage)
        return h

    def forward(self, step: StepBuffers, cache, *, prefill: bool, logits_rows: torch.Tensor | None = None,
                gather_logits: bool = True, return_hidden: bool = False):
        """Returns bf16 logits ``[rows, vocab]`` (all tokens, or ``logits_rows`` of them).  With tensor parallelism
        and ``gather_logits=False`` the result is this rank's vocabulary shard, for :meth:`sample_greedy`.
        ``return_hidden`` adds the residual stream of every token before the output norm (the MTP head's input)."""
        w = self.w
        self._begin_step()
        rows = step.input_ids.numel()
        if self._fused_tp(rows):
            # the residual stream lives in the collective's peer-mapped buffer, so finished rows can be pushed to it
            h0 = self.collective.stream_rows(self.cfg.hidden_size, rows)
            if h0.is_cuda:
                ops.embed(step.input_ids, w.embed, out=h0)
            else:
                h0.copy_(w.embed[step.input_ids.long()])
            h, x_head = self._run_layers_fused(h0, step, cache, prefill)
            hidden = h
            if logits_rows is None:
                with scope("head", h.device):
                    logits = w.lm_head(*x_head)
                    if gather_logits:
                        logits = self.collective.gather_columns(logits)
                return (logits, hidden) if return_hidden else logits
        else:
            h = self._run_layers(self._embed(step.input_ids), step, cache, prefill)
            hidden = h
        if logits_rows is not None:
            h = h[logits_rows.long()] if not h.is_cuda else h.index_select(0, logits_rows.long())
        logits = self._head(h, w.final_norm, gather_logits)
        return (logits, hidden) if return_hidden else logits

    def _begin_step(self) -> None:
        if self.tp > 1 and hasattr(self.collective, "begin_step"):
            self.collective.begin_step()

    def mtp_forward(self, step: StepBuffers, cache, hidden: torch.Tensor, *, prefill: bool,
                    logits_rows: torch.Tensor | None = None):
        """MTP head over the tokens of ``step``: row ``i`` pairs ``hidden[i]`` (the main model's, or the head's own
        previous output when drafts are chained) with the embedding of ``step.input_ids[i]`` -- the token that
        FOLLOWS that position -- and predicts the token after it.  The head's KV rows go to cache layer
        ``num_layers`` at ``step.slots``.  Returns (vocabulary-shard logits, the head's output hidden states)."""
        m = self.w.mtp
        eps = self.cfg.rms_eps
        self._begin_step()
        e = self._embed(step.input_ids)
        if e.is_cuda:
            _, _, ye, _ = ops.rmsnorm_quant(e, m.enorm, eps, want_q=False, want_y=True)
            _, _, yh, _ = ops.rmsnorm_quant(hidden, m.hnorm, eps, want_q=False, want_y=True)
        else:
            _, _, ye, _ = ref.rmsnorm_quant(e, m.enorm, eps)
            _, _, yh, _ = ref.rmsnorm_quant(hidden, m.hnorm, eps)
        zq, zs = self._quant(torch.cat([ye, yh], dim=1))
        h = m.eh_proj(zq, zs)
        h = self._block(h, m.layer, cache.layer(self.cfg.num_layers), step, prefill)
        out_hidden = h
        if logits_rows is not None:
            h = h[logits_rows.long()] if not h.is_cuda else h.index_select(0, logits_rows.long())
        return self._head(h, m.final_norm if m.final_norm is not None else self.w.final_norm, False), out_hidden

    def sample_greedy(self, logits: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        """Arg-max token per row.  Under TP ``logits`` is this rank's vocabulary shard (``gather_logits=False``)."""
        if self.tp > 1:
            return self.collective.argmax(logits, out)
        if logits.is_cuda:
            return ops.argmax(logits, out=out)
        res = logits.float().argmax(-1).to(torch.int32)
        if out is not None:
            out.copy_(res)
            return out
        return res
