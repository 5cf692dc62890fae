"""YaRN rotary scaling: the blend against a direct restatement, the import of Hugging Face keys, and the model path."""

import math

import torch

from mfq_b200.models.rope_scaling import YarnScaling
from mfq_b200.ops import reference as ref


def _direct(rot, theta, factor, original, beta_fast=32.0, beta_slow=1.0):
    """Per-pair loop written from the definition (no shared code with the module)."""
    out = []
    def corr(n):
        return rot * math.log(original / (n * 2 * math.pi)) / (2 * math.log(theta))
    low, high = max(math.floor(corr(beta_fast)), 0), min(math.ceil(corr(beta_slow)), rot - 1)
    for i in range(rot // 2):
        f = theta ** (-2 * i / rot)
        ramp = min(max((i - low) / (high - low), 0.0), 1.0)
        out.append((1 - ramp) * f + ramp * f / factor)
    return torch.tensor(out)


def test_blend_matches_the_definition_and_factor_one_is_plain_rope():
    y = YarnScaling(factor=4.0, original_max_position=4096)
    got = y.inv_freq(128, 1e4)
    torch.testing.assert_close(got, _direct(128, 1e4, 4.0, 4096).float(), rtol=2e-5, atol=0)
    base = YarnScaling().inv_freq(128, 1e4)
    assert torch.equal(got[:8], base[:8])  # the fastest pairs are untouched
    torch.testing.assert_close(got[-8:], base[-8:] / 4.0)  # the slowest are interpolated
    assert abs(y.mscale - (0.1 * math.log(4.0) + 1)) < 1e-12 and YarnScaling().mscale == 1.0
    f, low, high, m = y.kernel_args(128, 1e4)
    assert f == 4.0 and 0 <= low < high <= 127 and m == y.mscale
    x = torch.randn(5, 2, 128).bfloat16()
    pos = torch.tensor([0, 1, 100, 5000, 16000])
    assert torch.equal(ref.rope(x, pos, 1e4), ref.rope(x, pos, 1e4, None, YarnScaling()))
    scaled = ref.rope(x, pos, 1e4, None, y).float()
    assert torch.allclose(scaled[0], x[0].float() * y.mscale, rtol=1e-2, atol=1e-2)  # position 0: only the attention factor
    # rotations preserve the norm of every pair up to the attention factor
    torch.testing.assert_close(scaled.norm(dim=-1), x.float().norm(dim=-1) * y.mscale, rtol=1e-2, atol=1e-2)


def test_hf_keys():
    y = YarnScaling.from_hf({"max_position_embeddings": 131072, "rope_scaling": {
        "rope_type": "yarn", "factor": 4.0, "original_max_position_embeddings": 32768}})
    assert y.factor == 4.0 and y.original_max_position == 32768 and y.max_position() == 131072 and y.softmax_scale_factor == 1.0
    assert YarnScaling.from_hf({"rope_scaling": {"rope_type": "linear", "factor": 2.0}}) is None and YarnScaling.from_hf({}) is None
    d = YarnScaling.from_hf({"kv_lora_rank": 512, "max_position_embeddings": 163840, "rope_scaling": {
        "type": "yarn", "factor": 40, "original_max_position_embeddings": 4096, "beta_fast": 32, "beta_slow": 1,
        "mscale": 1.0, "mscale_all_dim": 1.0}})
    m = 0.1 * math.log(40) + 1
    assert abs(d.mscale - 1.0) < 1e-12 and abs(d.softmax_scale_factor - m * m) < 1e-9  # equal mscales cancel on cos / sin
    assert YarnScaling.from_dict(d.to_dict()) == d
    from mfq_b200.architectures import config_from_hf
    cfg = config_from_hf({"vocab_size": 100, "hidden_size": 64, "num_hidden_layers": 1, "num_attention_heads": 2,
                          "max_position_embeddings": 131072,
                          "rope_scaling": {"rope_type": "yarn", "factor": 4.0, "original_max_position_embeddings": 32768}})
    assert cfg["rope_scaling"]["factor"] == 4.0 and cfg["max_position"] == 131072


def test_model_path_uses_the_scaled_frequencies(tmp_path):
    """Same checkpoint with and without the extension: the first token (position 0 .. few) barely moves, far positions
    do; the engine runs beyond the trained context."""
    from mfq_b200.checkpoint import load_engine
    from mfq_b200.cli import main
    ckpt = tmp_path / "t.mfq"
    assert main(["quantize", "synthetic:tiny-moe-128", str(ckpt), "--full-precision"]) == 0
    plain, tok, cfg0 = load_engine(ckpt, "cpu", max_batch=1, max_seq_len=96)
    ext, _, cfg1 = load_engine(ckpt, "cpu", max_batch=1, max_seq_len=96, yarn_context_extension=4.0)
    assert cfg0.rope_scaling is None and cfg1.rope_scaling["factor"] == 4.0 and cfg1.max_position == 4 * cfg0.max_position
    assert ext.model.rope_scaling.factor == 4.0 and plain.model.rope_scaling is None
    ids = torch.arange(3, 67)
    a = plain.generate([ids], 4).tokens
    b = ext.generate([ids], 4).tokens
    assert a.shape == b.shape == (1, 4)
