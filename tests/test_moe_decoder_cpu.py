"""The FP8 MoE decoder (CPU reference path) against the plain fp32 MoE LM on the same checkpoint."""

import torch

from mfq_b200.engine.llm_engine import LLMEngine
from mfq_b200.evaluation.kld import compare_logits
from mfq_b200.models.llama import StepBuffers
from mfq_b200.models.moe_decoder import MoeDecoderConfig, MoeDecoderModel, MoeWeights
from mfq_b200.models.moe_lm import MoeConfig, MoeLM, dequantize_checkpoint, init_weights, quantize_moe_checkpoint


def configs():
    lm = MoeConfig(head_dim=128, hidden_size=256, moe_intermediate=128, shared_intermediate=128, num_experts=8, top_k=2)
    dec = MoeDecoderConfig(vocab_size=lm.vocab_size, hidden_size=256, num_layers=lm.num_layers, num_heads=lm.num_heads,
                           num_kv_heads=lm.num_kv_heads, head_dim=128, rope_theta=lm.rope_theta, rms_eps=lm.rms_eps,
                           num_experts=8, top_k=2, moe_intermediate=128, shared_intermediate=128)
    return lm, dec


def test_fp8_moe_decoder_tracks_fp32_model():
    lm_cfg, dec_cfg = configs()
    w = init_weights(lm_cfg, seed=2, std=0.05)
    q = quantize_moe_checkpoint(w, "NINT4,NVQ3,MXFP4")
    weights = MoeWeights.from_tensors(dec_cfg, q, "cpu")
    model = MoeDecoderModel(dec_cfg, weights)
    eng = LLMEngine(model, max_batch=1, max_seq_len=64, device="cpu")
    prompt = torch.randint(0, lm_cfg.vocab_size, (40,), generator=torch.Generator().manual_seed(5))
    eng.cache.assign(0, 0, 40)
    step = StepBuffers(input_ids=prompt.to(torch.int32), positions=torch.arange(40, dtype=torch.int32),
                       slots=eng.cache.slots(0, 0, 40), cu_seqlens=[0, 40])
    got = model.forward(step, eng.cache, prefill=True).float()
    want = MoeLM(lm_cfg, dequantize_checkpoint(q)).forward(prompt)
    r = compare_logits(want, got)
    assert r.kld < 0.02 and r.top1_agreement > 0.5, r  # near-flat random-init logits flip easily
    # and generation runs end to end through the engine
    out = LLMEngine(model, max_batch=1, max_seq_len=64, device="cpu").generate([prompt], 4)
    assert out.tokens.shape == (1, 4)


def test_native_4bit_loading_keeps_nint_codes():
    """NINT4 attention projections stay 4-bit (in-pipeline-decode GEMM) and predict like the FP8-transcoded model."""
    import torch
    import mfq_b200.quantize.expertwise as ew
    from mfq_b200.checkpoint import quantize_tensors
    from mfq_b200.engine.llm_engine import LLMEngine
    from mfq_b200.models.llama import StepBuffers, W4Linear
    from mfq_b200.models.moe_decoder import MoeDecoderConfig, MoeDecoderModel, MoeWeights
    from mfq_b200.models.moe_lm import MoeConfig, init_weights
    cfg = MoeDecoderConfig.tiny()
    t = init_weights(MoeConfig(head_dim=128, hidden_size=256, moe_intermediate=128, shared_intermediate=128), seed=4, std=0.05)
    old = ew._NINT_PRESETS[4]
    ew._NINT_PRESETS[4] = (32, 6)
    try:
        q = quantize_tensors({k: v.numpy() for k, v in t.items()}, dense="nint4")
    finally:
        ew._NINT_PRESETS[4] = old
    native = MoeWeights.from_tensors(cfg, q, "cpu", native_4bit=True)
    fp8 = MoeWeights.from_tensors(cfg, q, "cpu")
    assert isinstance(native.layers[0].qkv, W4Linear) and native.layers[0].qkv.w.n == (4 + 2 * 2) * 128
    assert not isinstance(fp8.layers[0].qkv, W4Linear)
    prompt = torch.randint(0, cfg.vocab_size, (20,), generator=torch.Generator().manual_seed(1))

    def logits(w):
        eng = LLMEngine(MoeDecoderModel(cfg, w), max_batch=1, max_seq_len=64, device="cpu")
        eng.cache.assign(0, 1, 20)
        step = StepBuffers(input_ids=prompt.int(), positions=torch.arange(20, dtype=torch.int32), slots=eng.cache.slots(1, 0, 20),
                           cu_seqlens=[0, 20])
        return eng.model.forward(step, eng.cache, prefill=True).float()
    a, b = logits(native), logits(fp8)
    scale = float(b.abs().max())
    assert float((a - b).abs().mean()) <= 0.03 * scale  # same checkpoint; FP8 transcoding vs exact 4-bit reconstruction


def test_native_layout_checkpoint_loads_without_requantizing(tmp_path):
    """A checkpoint written by ``optimize-layout`` holds E4M3 blocks: the loader adopts them bit for bit, and the model
    is the one the 4-bit source loads to (whose float values get the same FP8 blocks)."""
    import numpy as np
    import torch
    from mfq_b200 import formats as F
    from mfq_b200.cli import main
    from mfq_b200.formats.fp8sq import Fp8SqTensor
    from mfq_b200.models.moe_decoder import MoeDecoderConfig, MoeWeights
    src, dst = tmp_path / "q4.mfq", tmp_path / "native.mfq"
    assert main(["quantize", "synthetic:tiny-moe-128", str(src), "--bits", "4"]) == 0
    assert main(["optimize-layout", "--input", str(src), "--output", str(dst)]) == 0
    import json
    with F.open_mfq(dst) as store:
        cfg_d = json.loads(store.assets()["model_config.json"])
        cfg = MoeDecoderConfig(**{k: v for k, v in cfg_d.items() if k in MoeDecoderConfig.__dataclass_fields__})
        t = store["model.block.0.attention.query.weight"]
        assert isinstance(t, Fp8SqTensor)
        native = MoeWeights.from_tensors(cfg, store, "cpu")
        assert np.array_equal(native.layers[0].qkv.q.view(torch.uint8)[: t.shape[0]].numpy(), t.codes)
    with F.open_mfq(src) as store:
        source = MoeWeights.from_tensors(cfg, store, "cpu")
    assert torch.equal(native.layers[0].qkv.q.view(torch.uint8), source.layers[0].qkv.q.view(torch.uint8))
    assert torch.allclose(native.layers[1].o_proj.scale, source.layers[1].o_proj.scale, rtol=1e-6)
