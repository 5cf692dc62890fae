"""Packed expert weights on the GPU: in-register decode (NINT 1..8 bit, MXFP4) against the exact host reconstruction."""

import numpy as np
import pytest
import torch

from mfq_b200.formats import nint
from mfq_b200.ops import moe as moe_ops
from mfq_b200.ops import packed
from mfq_b200.quantize.mxfp4 import quantize_mxfp4
from mfq_b200.quantize.nint import quantize_nint
from gpu_common import assert_close, check_status, require_gpu_lib

pytestmark = pytest.mark.gpu


def _experts(n, k, specs, seed, min_units=0):
    rng = np.random.default_rng(seed)
    mats, dense = [], []
    units = max([min_units] + [int(np.ceil(np.ceil(k / gs) * gs / 128)) for _b, gs in specs if _b != 16] + [int(np.ceil(k / 128))])
    for bits, gs in specs:
        w = (rng.standard_normal((n, k)) * 0.05).astype(np.float32)
        if bits == 16:
            m = packed.pack_mxfp4(quantize_mxfp4(w), min_units=units)
        else:
            m = packed.pack_nint(quantize_nint(w, nint.NintSpec(bits=bits, groupsize=gs, sub_bits=6)), min_units=units)
        mats.append(m)
        dense.append(packed.dequantize(m))
    return mats, np.stack(dense)


@pytest.mark.parametrize("gs", [16, 24, 32])
def test_gpu_decode_matches_host_reconstruction(gs):
    require_gpu_lib()
    specs = [(b, gs) for b in (1, 2, 3, 4, 5, 6, 7, 8)] + [(16, 32)]
    mats, dense = _experts(48, 416, specs, seed=gs)
    pe = packed.PackedExperts(mats, "cuda")
    for e in range(len(specs)):
        got = pe.dense(e).float().cpu()
        # weights are evaluated as q * s - m in bf16 arithmetic: 2^-9 relative on s and on m (which is several code steps
        # wide), then on the result; where q * s and m nearly cancel a few elements exceed the element-wise bound
        assert_close(got, torch.from_numpy(dense[e]), rel=3e-2, what=f"decode of width code {specs[e][0]}", outliers=2e-2)
    check_status()


@pytest.mark.parametrize("tokens,k_in,n_out", [(1, 256, 64), (5, 416, 96), (40, 2048, 128), (16, 512, 2048)])
def test_grouped_product_matches_reference(tokens, k_in, n_out):
    require_gpu_lib()
    specs = [(2, 24), (3, 24), (4, 24), (6, 24), (16, 32), (5, 24)]
    mats, dense = _experts(n_out, k_in, specs, seed=tokens)
    pe = packed.PackedExperts(mats, "cuda")
    g = torch.Generator(device="cuda").manual_seed(tokens)
    top_k = 3
    x = torch.randn((tokens, k_in), generator=g, device="cuda").to(torch.bfloat16)
    ids = torch.stack([torch.randperm(len(specs), generator=g, device="cuda")[:top_k] for _ in range(tokens)]).to(torch.int32)
    plan = moe_ops.plan_routes(ids, 0, len(specs), token_tile=16)
    got = packed.packed_gemv_grouped(pe, x, plan, gather=True)
    check_status()
    rows = int(plan.totals[0])
    assert rows == tokens * top_k
    offsets, src = plan.offsets.cpu().numpy(), plan.src_token.cpu().numpy()
    w = torch.from_numpy(dense).cuda()
    want = torch.zeros((rows, n_out), device="cuda")
    for e in range(len(specs)):
        for r in range(offsets[e], offsets[e + 1]):
            want[r] = w[e] @ x[src[r]].float()
    assert_close(got[:rows].float(), want, rel=3e-2, what="grouped packed product")
    # sorted-row input (the down projection's form)
    xs = x[torch.from_numpy(src[:rows]).long().cuda()].contiguous()
    got2 = packed.packed_gemv_grouped(pe, xs, plan, gather=False)
    assert torch.equal(got2[:rows], got[:rows])


def test_packed_moe_layer_matches_reference():
    require_gpu_lib()
    hidden, inter, e, top_k, tokens = 256, 128, 6, 2, 9
    specs = [(3, 24), (4, 24), (2, 24), (16, 32), (5, 24), (6, 24)]
    gu_m, gu = _experts(2 * inter, hidden, specs, seed=1)
    dn_m, dn = _experts(hidden, inter, specs[::-1], seed=2)
    pgu, pdn = packed.PackedExperts(gu_m, "cuda"), packed.PackedExperts(dn_m, "cuda")
    g = torch.Generator(device="cuda").manual_seed(5)
    x = torch.randn((tokens, hidden), generator=g, device="cuda").to(torch.bfloat16)
    base = torch.randn((tokens, hidden), generator=g, device="cuda").to(torch.bfloat16)
    ids = torch.stack([torch.randperm(e, generator=g, device="cuda")[:top_k] for _ in range(tokens)]).to(torch.int32)
    wt = torch.rand((tokens, top_k), generator=g, device="cuda")
    got = packed.moe_ffn_packed(x, ids, wt, pgu, pdn, base=base)
    check_status()
    want = base.float().clone()
    gu_t, dn_t = torch.from_numpy(gu).cuda(), torch.from_numpy(dn).cuda()
    for t in range(tokens):
        for j in range(top_k):
            ex = int(ids[t, j])
            a = (gu_t[ex] @ x[t].float()).to(torch.bfloat16).float()
            h = (torch.nn.functional.silu(a[:inter]) * a[inter:]).to(torch.bfloat16).float()
            want[t] += wt[t, j] * (dn_t[ex] @ h).to(torch.bfloat16).float()
    assert_close(got.float(), want, rel=3e-2, what="packed MoE layer")


def test_synthetic_payloads_decode_to_the_requested_spread():
    require_gpu_lib()
    pe = packed.PackedExperts.synthetic(4, 64, 512, [2, 3, 4, 16], "cuda", gs=32, seed=3, std=0.02)
    for e in range(4):
        w = pe.dense(e).float()
        assert torch.isfinite(w).all() and 0.005 < float(w.std()) < 0.08, (e, float(w.std()))
    assert 2.0 < pe.bits_per_weight() < 5.0


def test_checkpoint_experts_stay_packed_and_match_the_fp8_transcode():
    """A checkpoint whose routed experts are MFE pools of NINT4 / NINT3 / MXFP4 loads with the experts kept in their
    packed codes; its logits agree with the same checkpoint transcoded to FP8 at load time, and graph decode works."""
    require_gpu_lib()
    from mfq_b200.engine.llm_engine import LLMEngine
    from mfq_b200.evaluation.kld import compare_logits
    from mfq_b200.models.llama import StepBuffers
    from mfq_b200.models.moe_decoder import MoeDecoderConfig, MoeDecoderModel, MoeWeights
    from mfq_b200.models.moe_lm import MoeConfig, init_weights, quantize_moe_checkpoint
    cfg = MoeDecoderConfig.tiny()
    ck = quantize_moe_checkpoint(init_weights(MoeConfig(head_dim=128, hidden_size=256, moe_intermediate=128,
                                                        shared_intermediate=128), seed=9, std=0.05), "NINT4,NINT3,MXFP4")
    prompt = torch.randint(0, cfg.vocab_size, (50,), generator=torch.Generator().manual_seed(2))
    outs = {}
    for packed_mode in (False, True):
        w = MoeWeights.from_tensors(cfg, ck, "cuda", packed_experts=packed_mode)
        assert (w.layers[0].moe.packed_gate_up is not None) == packed_mode
        model = MoeDecoderModel(cfg, w)
        eng = LLMEngine(model, max_batch=2, max_seq_len=96, use_graphs=False)
        eng.cache.assign(0, 0, 50)
        step = StepBuffers(input_ids=prompt.cuda().int(), positions=torch.arange(50, dtype=torch.int32, device="cuda"),
                           slots=eng.cache.slots(0, 0, 50).cuda(), cu_seqlens=[0, 50])
        outs[packed_mode] = model.forward(step, eng.cache, prefill=True).float().cpu()
    check_status()
    r = compare_logits(outs[False], outs[True])
    assert r.kld < 0.01 and r.top1_agreement > 0.8, r
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=torch.Generator().manual_seed(n)) for n in (17, 40)]
    a = LLMEngine(model, max_batch=2, max_seq_len=96, use_graphs=False).generate(prompts, 8)
    b = LLMEngine(model, max_batch=2, max_seq_len=96, use_graphs=True).generate(prompts, 8)
    assert torch.equal(a.tokens, b.tokens)
    # the packed experts occupy about half a byte per weight, not the full byte of the transcode
    pgu = w.layers[0].moe.packed_gate_up
    assert pgu.bits_per_weight() < 7.5, pgu.bits_per_weight()  # 256-wide rows padded to whole 128-code units
    check_status()


def test_palette_coded_mxfp4_experts_run_on_the_packed_mxfp4_path():
    """MXFP4-SQ expert pools (rows of 1..4 symbol bits over catalogue palettes) decode to legal MXFP4 at load: the
    packed kernels run them, and the logits are bit-equal to those of the same checkpoint with the pools expanded to
    plain MXFP4 beforehand."""
    require_gpu_lib()
    from mfq_b200.engine.llm_engine import LLMEngine
    from mfq_b200.formats.mfe import MfePool, MfeTensor
    from mfq_b200.formats.mx import MxTensor
    from mfq_b200.formats.mxfp4sq import Mxfp4SqTensor, to_mxfp4
    from mfq_b200.models.llama import StepBuffers
    from mfq_b200.models.moe_decoder import MoeDecoderConfig, MoeDecoderModel, MoeWeights
    from mfq_b200.models.moe_lm import MoeConfig, init_weights, quantize_moe_checkpoint
    from mfq_b200.quantize.mxfp4_sq import quantize_mxfp4_sq
    cfg = MoeDecoderConfig.tiny()
    ck = quantize_moe_checkpoint(init_weights(MoeConfig(head_dim=128, hidden_size=256, moe_intermediate=128,
                                                        shared_intermediate=128), seed=11, std=0.05), "MXFP4")
    coded, plain = dict(ck), dict(ck)
    pools = 0
    for name, t in ck.items():
        if isinstance(t, MfeTensor):
            sq = tuple(MfePool(p.expert_ids, quantize_mxfp4_sq(p.tensor, target_bits=3.0), p.runtime) for p in t.pools)
            coded[name] = MfeTensor(t.shape, sq)
            plain[name] = MfeTensor(t.shape, tuple(MfePool(p.expert_ids, to_mxfp4(p.tensor), p.runtime) for p in sq))
            pools += len(sq)
            assert all(isinstance(p.tensor, Mxfp4SqTensor) for p in sq) and all(isinstance(p.tensor, MxTensor) for p in plain[name].pools)
    assert pools > 0
    prompt = torch.randint(0, cfg.vocab_size, (40,), generator=torch.Generator().manual_seed(5))
    outs = []
    for tensors in (coded, plain):
        w = MoeWeights.from_tensors(cfg, tensors, "cuda", packed_experts=True)
        assert w.layers[0].moe.packed_gate_up is not None
        model = MoeDecoderModel(cfg, w)
        eng = LLMEngine(model, max_batch=2, max_seq_len=96, use_graphs=False)
        eng.cache.assign(0, 0, 40)
        step = StepBuffers(input_ids=prompt.cuda().int(), positions=torch.arange(40, dtype=torch.int32, device="cuda"),
                           slots=eng.cache.slots(0, 0, 40).cuda(), cu_seqlens=[0, 40])
        outs.append(model.forward(step, eng.cache, prefill=True).float().cpu())
    check_status()
    assert torch.equal(outs[0], outs[1])
