"""Python entry points of the CUDA kernels.  All tensors must live on the current CUDA device and be
contiguous; outputs may be preallocated (needed under CUDA-graph capture) or are allocated here."""

from __future__ import annotations

import math
import os

import torch

from .lib import Workspace, check, lib, ptr, stream_ptr

FP8 = torch.float8_e4m3fn


GEMV_MAX_ROWS = 8   # up to this many rows the weight-streaming kernel (fp8_gemv.cu) always replaces the tcgen05 GEMM
GEMV_MID_ROWS = 16  # ... up to this many when the matrix is at most GEMV_MID_WEIGHTS values
GEMV_MID_WEIGHTS = 20 << 20
GEMV_WIDE_ROWS = 64  # ... and up to this many when the weight matrix is small (see use_gemv)


def gemv_enabled() -> bool:
    """``MFQ_GEMV=0`` in the environment sends every shape through the tcgen05 GEMM (A/B measurements)."""
    from ..config import current
    return current().gemv


def use_gemv(m: int, n: int, k: int) -> bool:
    """Whether ``[m, k] x [n, k]^T`` goes to the weight-streaming kernel: always for up to 8 rows; for 9..16 rows only
    for matrices up to 20 M values (measured at 16 rows on B200, this kernel / tcgen05: o_proj 4096 x 4096 7.0 / 10.4 us,
    but gate_up 28672 x 4096 44.5 / 22.7, down 24.0 / 18.3, LM head 168 / 92 -- a second 8-column block doubles its MMA
    work while the tcgen05 tile is still nearly free); for up to 64 rows only when the output is a few tiles wide and the
    matrix small (a tensor-parallel rank's q/k/v shard), where the tcgen05 path would need a deep split-K whose reduction
    costs more than the product: 768 x 4096 at 64 rows takes 11.1 us here against 14.7 us there; from 3072 x 4096 up the
    tcgen05 path wins (the legacy ``mma.sync`` pipe this kernel uses runs at a fraction of the tcgen05 rate)."""
    if n % 16 or not gemv_enabled():
        return False
    if m <= GEMV_MAX_ROWS:
        return True
    if m <= GEMV_MID_ROWS and n * k <= GEMV_MID_WEIGHTS:
        return True
    return m <= GEMV_WIDE_ROWS and n <= 1024 and n * k <= (4 << 20)


def _token_tile(m: int) -> int:
    return 16 if m <= 16 else 32 if m <= 32 else 64 if m <= 64 else 128


def pick_splits(m: int, n: int, k: int, sms: int = 148) -> int:
    """Split-K factor minimizing a wave model of the weight-streaming GEMM.

    cost(s) = waves(s) * (K blocks per CTA + fixed ramp of ~4 blocks) + a small charge for the reduction;
    it fills the SMs when the (n, token) tile grid alone cannot and avoids a nearly empty last wave.
    """
    tiles = math.ceil(n / 128) * math.ceil(m / _token_tile(m))
    kb = k // 128
    if tiles >= 4 * sms or kb <= 1:
        return 1
    if m <= 64 and (tiles, kb) in _MEASURED_SPLITS:
        return _MEASURED_SPLITS[(tiles, kb)]
    best, best_cost = 1, None
    # Up to 8 splits meet in a cluster's shared memory; more would fall back to the global scratch buffer with a
    # last-arriver sum, which costs several microseconds (1536 x 4096 at 64 rows: 14.7 us with 11 splits, 9.1 with 8), so
    # decode-sized tiles never ask for more.  A cluster grid that needs nearly every SM (129..148 CTAs) does not place
    # well -- clusters stay inside a GPC -- and is charged for it.
    small = _token_tile(m) <= 64
    for s in range(1, min(kb, 8 if small else 16) + 1):
        per = math.ceil(kb / s)
        if s > 1 and per < 2:
            break
        ctas = tiles * math.ceil(kb / per)
        cost = math.ceil(ctas / sms) * (per + 4) + (1.5 if s > 1 else 0.0)
        if small and s > 1 and 128 < ctas <= sms:
            cost += 3.0
        if best_cost is None or cost < best_cost - 1e-9:
            best, best_cost = s, cost
    return best


# Decode shapes where a sweep inside a decode step disagrees with the wave model, (output tiles, K blocks) -> splits:
# 48 tiles x 32 blocks (6144 x 4096, the fused q/k/v projection of an 8B model) takes 17.4 us with the model's 3 splits --
# 144 CTAs in clusters of 3 leave no slack for cluster placement -- and 14.6 us with 4.
_MEASURED_SPLITS = {(48, 32): 4}

PAIR_MIN_ROWS = 1024  # batches at least this wide take the two-SM GEMM (``csrc/fp8_gemm_2cta.cu``)


def pair_tile(m: int, n: int) -> int:
    """Token tile of the two-SM GEMM for this shape, 0 = use the one-SM kernel.  ``MFQ_GEMM_PAIR`` = 0 / 128 / 256
    overrides the choice."""
    forced = os.environ.get("MFQ_GEMM_PAIR")
    tile = int(forced) if forced not in (None, "") else _PAIR_DEFAULT
    if tile not in (128, 256) or n % 256 or m < PAIR_MIN_ROWS:
        return 0
    return tile


_PAIR_DEFAULT = 0


def fp8_gemm(x_q: torch.Tensor, x_scale: torch.Tensor, w_q: torch.Tensor, w_scale: torch.Tensor, *,
             out: torch.Tensor | None = None, residual: torch.Tensor | None = None, splits: int | None = None,
             token_tile: int | None = None, pair: int | None = None) -> torch.Tensor:
    """``out[M, N] = (x_q * x_scale[:, None]) @ (w_q * blockscale(w_scale)).T`` in bf16 (+ residual).
    ``pair``: token tile (128 / 256) of the two-SM kernel, 0 = never, None = by shape (:func:`pair_tile`)."""
    m, k = x_q.shape
    n = w_q.shape[0]
    assert w_q.shape[1] == k and k % 128 == 0 and x_q.dtype == FP8 and w_q.dtype == FP8
    assert x_scale.dtype == torch.float32 and w_scale.dtype == torch.float32 and x_scale.numel() == m
    assert w_scale.shape == (math.ceil(n / 128), k // 128) and w_scale.is_contiguous()
    if out is None:
        out = torch.empty((m, n), dtype=torch.bfloat16, device=x_q.device)
    if splits is None and token_tile is None and use_gemv(m, n, k):
        rc = lib().mfq_fp8_gemv(ptr(w_q), ptr(w_scale), ptr(x_q), ptr(x_scale), ptr(out), ptr(residual), m, n, k, stream_ptr())
        check(rc, "fp8_gemv")
        return out
    ws = Workspace.get(x_q.device)
    if pair is None:
        pair = pair_tile(m, n) if splits is None and token_tile is None else 0
    if pair:
        assert pair in (128, 256) and n % 256 == 0
        rc = lib().mfq_fp8_gemm_pair(ptr(w_q), ptr(w_scale), ptr(x_q), ptr(x_scale), ptr(out), ptr(residual), ptr(ws.status),
                                     m, n, k, pair, stream_ptr())
        check(rc, "fp8_gemm_pair")
        return out
    bt = token_tile or _token_tile(m)
    sp = pick_splits(m, n, k) if splits is None else splits
    rc = lib().mfq_fp8_gemm(ptr(w_q), ptr(w_scale), ptr(x_q), ptr(x_scale), ptr(out), ptr(residual), ptr(ws.splitk),
                            ws.splitk.numel(), ptr(ws.counters), ws.counters.numel(), ptr(ws.status), m, n, k, bt, sp,
                            stream_ptr())
    check(rc, "fp8_gemm")
    return out


def rmsnorm_quant(x: torch.Tensor, weight: torch.Tensor, eps: float, *, residual: torch.Tensor | None = None,
                  want_q: bool = True, want_y: bool = False, q_out=None, scale_out=None, y_out=None,
                  residual_out=None):
    """(x [+ residual]) -> RMSNorm -> fp8 rows.  Returns ``(q, scale, y, new_residual)`` (unused ones None)."""
    m, h = x.shape
    dev = x.device
    if want_q:
        q_out = torch.empty((m, h), dtype=FP8, device=dev) if q_out is None else q_out
        scale_out = torch.empty(m, dtype=torch.float32, device=dev) if scale_out is None else scale_out
    if want_y and y_out is None:
        y_out = torch.empty_like(x)
    if residual is not None and residual_out is None:
        residual_out = torch.empty_like(x)
    rc = lib().mfq_rmsnorm_quant(ptr(x), ptr(residual), ptr(residual_out), ptr(weight), ptr(q_out), ptr(scale_out),
                                 ptr(y_out), m, h, float(eps), stream_ptr())
    check(rc, "rmsnorm_quant")
    return q_out, scale_out, y_out, residual_out


ACT_GEMV_MAX_ROWS = 4  # rows up to which a projection rebuilds its FP8 activations itself (fp8_gemv_act_kernel)
ACT_NORM, ACT_PLAIN, ACT_SWIGLU = 0, 1, 2


def act_gemv_ok(m: int, n: int, k: int) -> bool:
    """Whether ``fp8_gemv_act`` takes this shape: a handful of rows, rows of at most 16384 values (64 KB of FP8 rows
    in shared memory), and the standalone norm kernel's layout must be one this kernel can replay (<= 512 threads)."""
    return gemv_enabled() and 0 < m <= ACT_GEMV_MAX_ROWS and n % 16 == 0 and k % 128 == 0 and k <= 16384


ACT_GEMV_MAX_CTAS = 296  # one wave at two CTAs per SM


def act_gemv_pays(m: int, n: int, k: int) -> bool:
    """Whether a model should fold the preparation in.  Measured on B200 with one row (Llama-8B, 2.75 ms per step with
    the standalone kernels): all four projections of a layer folded 3.23 ms -- every CTA repeats the preparation, so the
    1792-CTA gate/up product pays it once per wave, six times; only the single-wave projections (o_proj, down) folded
    2.92 ms -- three dependent passes over the row with block-wide reductions in between cost more inside every CTA than
    the hand-over to a separate one-CTA kernel.  So the answer is no unless ``MFQ_ACT_GEMV=1`` asks for it; the kernel
    stays for shapes and parts where the balance differs."""
    from ..config import current
    return current().act_gemv and act_gemv_ok(m, n, k) and n // 16 <= ACT_GEMV_MAX_CTAS


def fp8_gemv_act(x: torch.Tensor, w_q: torch.Tensor, w_scale: torch.Tensor, mode: int, *, norm_w: torch.Tensor | None = None,
                 eps: float = 0.0, residual: torch.Tensor | None = None, out: torch.Tensor | None = None) -> torch.Tensor:
    """``out = W . quant(prep(x))`` (+ residual) for up to 4 bf16 rows, the preparation -- RMSNorm * ``norm_w``
    (``ACT_NORM``), nothing (``ACT_PLAIN``) or ``silu(x[:, :K]) * x[:, K:]`` (``ACT_SWIGLU``) -- and the per-row FP8
    quantization done inside the product kernel, bit-identical to the standalone kernels followed by ``fp8_gemm``'s
    weight-streaming path."""
    m = x.shape[0]
    n, k = w_q.shape
    assert x.dtype == torch.bfloat16 and x.stride(1) == 1 and x.shape[1] == (2 * k if mode == ACT_SWIGLU else k)
    assert act_gemv_ok(m, n, k) and (mode != ACT_NORM or norm_w is not None)
    if out is None:
        out = torch.empty((m, n), dtype=torch.bfloat16, device=x.device)
    rc = lib().mfq_fp8_gemv_act(ptr(w_q), ptr(w_scale), ptr(x), x.stride(0), ptr(norm_w), float(eps), ptr(out), ptr(residual),
                                m, n, k, mode, stream_ptr())
    check(rc, "fp8_gemv_act")
    return out


def quant_rows(x: torch.Tensor, *, q_out=None, scale_out=None):
    m, k = x.shape
    q_out = torch.empty((m, k), dtype=FP8, device=x.device) if q_out is None else q_out
    scale_out = torch.empty(m, dtype=torch.float32, device=x.device) if scale_out is None else scale_out
    check(lib().mfq_quant_rows(ptr(x), ptr(q_out), ptr(scale_out), m, k, x.stride(0), 0, stream_ptr()), "quant_rows")
    return q_out, scale_out


def silu_mul_quant(gate_up: torch.Tensor, *, q_out=None, scale_out=None):
    """``[M, 2I]`` (gate | up) -> fp8 ``silu(gate) * up`` rows ``[M, I]`` + per-row multiplier."""
    m, two_i = gate_up.shape
    i = two_i // 2
    q_out = torch.empty((m, i), dtype=FP8, device=gate_up.device) if q_out is None else q_out
    scale_out = torch.empty(m, dtype=torch.float32, device=gate_up.device) if scale_out is None else scale_out
    check(lib().mfq_quant_rows(ptr(gate_up), ptr(q_out), ptr(scale_out), m, i, gate_up.stride(0), 1, stream_ptr()),
          "silu_mul_quant")
    return q_out, scale_out


def silu_mul(gate_up: torch.Tensor) -> torch.Tensor:
    """``[M, 2I]`` (gate | up) -> bf16 ``silu(gate) * up`` ``[M, I]`` (input of the bf16-activation GEMMs)."""
    m, two_i = gate_up.shape
    out = torch.empty((m, two_i // 2), dtype=torch.bfloat16, device=gate_up.device)
    check(lib().mfq_silu_mul_bf16(ptr(gate_up), ptr(out), m, two_i // 2, gate_up.stride(0), stream_ptr()), "silu_mul")
    return out


def gate_quant_rows(x: torch.Tensor, gate: torch.Tensor):
    """fp8 rows of ``x * sigmoid(gate)`` (+ per-row multipliers); ``gate`` may be a strided column slice."""
    m, k = x.shape
    q_out = torch.empty((m, k), dtype=FP8, device=x.device)
    scale_out = torch.empty(m, dtype=torch.float32, device=x.device)
    check(lib().mfq_gate_quant_rows(ptr(x), ptr(gate), ptr(q_out), ptr(scale_out), m, k, x.stride(0), gate.stride(0),
                                    stream_ptr()), "gate_quant_rows")
    return q_out, scale_out


def rope_kv_write(qkv: torch.Tensor, positions: torch.Tensor, slots: torch.Tensor, kv, *, n_q: int, n_kv: int,
                  head_dim: int, theta: float, rot: int | None = None, q_out=None, kd_out=None,
                  vd_out=None, q_norm: torch.Tensor | None = None, k_norm: torch.Tensor | None = None,
                  norm_eps: float = 1e-6, scaling=None) -> torch.Tensor:
    """Rotate Q/K, write K/V of each token into the fp8 page pool ``kv`` (a :class:`LayerKV`).  ``scaling``: a
    :class:`~mfq_b200.models.rope_scaling.YarnScaling` for context extension.  ``kd_out`` /
    ``vd_out`` (``[T, Hk, D]`` bf16) optionally receive the values the pages now hold, for the chunk's attention.
    ``q_norm`` / ``k_norm`` (``[D]`` fp32): per-head RMSNorm before the rotation; ``rot`` < D: partial rotary.
    Rows of ``qkv`` may be wider than the q|k|v heads (e.g. an output gate after v); the row stride is honoured."""
    t = qkv.shape[0]
    q_out = torch.empty((t, n_q, head_dim), dtype=torch.bfloat16, device=qkv.device) if q_out is None else q_out
    if scaling is not None and (scaling.factor != 1.0 or scaling.mscale != 1.0):
        rc = lib().mfq_rope_kv_write_yarn(ptr(qkv), ptr(positions), ptr(slots), ptr(q_out), ptr(kv.k), ptr(kv.v), ptr(kv.k_scale),
                                          ptr(kv.v_scale), t, n_q, n_kv, head_dim, kv.page_size, rot or head_dim, float(theta),
                                          ptr(kd_out), ptr(vd_out), ptr(q_norm), ptr(k_norm), float(norm_eps), qkv.stride(0),
                                          *scaling.kernel_args(rot or head_dim, float(theta)), stream_ptr())
        check(rc, "rope_kv_write")
        return q_out
    rc = lib().mfq_rope_kv_write_ex(ptr(qkv), ptr(positions), ptr(slots), ptr(q_out), ptr(kv.k), ptr(kv.v), ptr(kv.k_scale),
                                    ptr(kv.v_scale), t, n_q, n_kv, head_dim, kv.page_size, rot or head_dim, float(theta),
                                    ptr(kd_out), ptr(vd_out), ptr(q_norm), ptr(k_norm), float(norm_eps), qkv.stride(0),
                                    stream_ptr())
    check(rc, "rope_kv_write")
    return q_out


def attn_splits_for(batch: int, kv_heads: int, ctx_len: int, head_dim: int = 128, rows: int = 1) -> int:
    """KV splits per (sequence, KV head) for the decode attention, fitted to sweeps on B200 (batch 1..128, contexts
    1k/4k/16k, 8 and 2 KV heads, head widths 128 and 256).  ``rows`` = query heads per KV head x query tokens per
    sequence.  Up to 8 rows run the tokens-as-rows kernel, 4 CTAs per SM (2 at width 256): the best split count is the
    largest one whose grid still fits one wave, with at least 256 tokens per split and at most 32 splits -- partial
    waves cost more than short splits, and a batch that fills the GPU by itself is not split at all.  Wider windows run
    the 16-row kernel at 3 CTAs per SM, where several waves of shorter CTAs (about 1300 tokens each) measured best."""
    n = max(1, batch * kv_heads)
    if rows > 8:
        by_ctas = -(-256 // n)
        by_len = int(ctx_len / 1300 + 0.5)
        return max(1, min(max(by_ctas, by_len), max(1, ctx_len // 256), 64))
    slots = 148 * (4 if head_dim <= 128 else 2)
    return max(1, min(slots // n, ctx_len // 256, 32))


def paged_attn_decode(q: torch.Tensor, kv, block_table: torch.Tensor, seq_lens: torch.Tensor, *, sm_scale: float,
                      splits: int = 1, q_len: int = 1, out=None) -> torch.Tensor:
    """``q [B*q_len, Hq, D]`` against the paged fp8 cache; ``seq_lens`` count the query tokens too."""
    rows, hq, d = q.shape
    b = rows // q_len
    hk = kv.k.shape[1]
    out = torch.empty_like(q) if out is None else out
    ws = Workspace.get(q.device)
    if splits > 1:
        assert rows * hq * splits * d <= ws.attn_acc.numel() and rows * hq * splits * 2 <= ws.attn_ml.numel()
    rc = lib().mfq_paged_attn_decode_mma(ptr(q), ptr(kv.k), ptr(kv.v), ptr(kv.k_scale), ptr(kv.v_scale),
                                         ptr(block_table), ptr(seq_lens), ptr(out), ptr(ws.attn_acc), ptr(ws.attn_ml), b,
                                         hq, hk, d, block_table.shape[1], float(sm_scale), splits, q_len,
                                         ptr(ws.status), stream_ptr())
    check(rc, "paged_attn_decode", 2 if splits > 1 else 1)
    return out


def argmax(logits: torch.Tensor, *, out=None) -> torch.Tensor:
    b, v = logits.shape
    out = torch.empty(b, dtype=torch.int32, device=logits.device) if out is None else out
    check(lib().mfq_argmax(ptr(logits), ptr(out), b, v, logits.stride(0), stream_ptr()), "argmax")
    return out


def embed(ids: torch.Tensor, table: torch.Tensor, *, out=None) -> torch.Tensor:
    t, h = ids.numel(), table.shape[1]
    out = torch.empty((t, h), dtype=torch.bfloat16, device=table.device) if out is None else out
    check(lib().mfq_embed(ptr(ids), ptr(table), ptr(out), t, h, stream_ptr()), "embed")
    return out


def decode_advance(sampled, input_ids, positions, seq_lens, slots, block_table, page_size: int, active=None) -> None:
    b = input_ids.numel()
    check(lib().mfq_decode_advance(ptr(sampled), ptr(input_ids), ptr(positions), ptr(seq_lens), ptr(slots),
                                   ptr(block_table), b, block_table.shape[1], page_size, ptr(active), stream_ptr()),
          "decode_advance")


def attn_prefill_bf16(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, sm_scale: float, *, out=None) -> torch.Tensor:
    """Causal attention of one sequence chunk on the tcgen05 kernels: ``q [T, Hq, D]``, ``k/v [Tk, Hk, D]`` (D 128 or
    256) with ``Tk >= T``: the first ``Tk - T`` keys are the sequence's past, query ``i`` sees keys ``0 .. i + (Tk - T)``."""
    t, hq, d = q.shape
    out = torch.empty_like(q) if out is None else out
    ws = Workspace.get(q.device)
    if d == 256:
        rc = lib().mfq_attn_prefill_d256(ptr(q), ptr(k), ptr(v), ptr(out), t, k.shape[0], hq, k.shape[1], float(sm_scale),
                                         ptr(ws.status), stream_ptr())
        check(rc, "attn_prefill_d256")
        return out
    rc = lib().mfq_attn_prefill_past(ptr(q), ptr(k), ptr(v), ptr(out), t, k.shape[0], hq, k.shape[1], d, float(sm_scale),
                                     ptr(ws.status), stream_ptr())
    check(rc, "attn_prefill_bf16")
    return out


def kv_gather_dequant(kv, block_row: torch.Tensor, tokens: int):
    """The first ``tokens`` cached K/V rows of one sequence (its page ids in ``block_row``) as bf16 ``[tokens, Hk, D]``."""
    hk, d = kv.k.shape[1], kv.k.shape[2] * kv.k.shape[4]
    kd = torch.empty((tokens, hk, d), dtype=torch.bfloat16, device=block_row.device)
    vd = torch.empty_like(kd)
    check(lib().mfq_kv_gather_dequant(ptr(kv.k), ptr(kv.v), ptr(kv.k_scale), ptr(kv.v_scale), ptr(block_row), ptr(kd), ptr(vd),
                                      tokens, hk, d, kv.page_size, stream_ptr()), "kv_gather_dequant")
    return kd, vd


def attn_prefill(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cu_seqlens: list[int], sm_scale: float) -> torch.Tensor:
    """Causal self-attention over a packed chunk (each sequence attends to itself)."""
    out = torch.empty_like(q)
    for i in range(len(cu_seqlens) - 1):
        a, b = cu_seqlens[i], cu_seqlens[i + 1]
        attn_prefill_bf16(q[a:b], k[a:b], v[a:b], sm_scale, out=out[a:b])
    return out
