"""Named profiling scopes: off by default, filterable, reported per name; the model and engine carry the call sites."""

import io

import pytest
import torch

from mfq_b200.utils import profiler as P


def test_scopes_accumulate_and_filter():
    p = P.Profiler(enabled=True, name_filter="ffn,head")
    for _ in range(3):
        with p.scope("ffn.down"):
            sum(range(1000))
    with p.scope("attn.qkv"):  # filtered out
        pass
    assert p.measure("head", lambda a, b: a + b, 2, 3) == 5
    items = {it.name: it for it in p.items()}
    assert set(items) == {"ffn.down", "head"} and items["ffn.down"].calls == 3 and items["ffn.down"].wall_ms > 0
    buf = io.StringIO()
    lines = p.report(buf)
    assert lines[0].startswith("profile_item name=ffn.down calls=3 cuda_ms=0.000 wall_ms=") and buf.getvalue().count("\n") == 2
    p.reset()
    assert p.items() == []


def test_disabled_profiler_records_nothing_and_env_is_validated():
    p = P.Profiler()
    with p.scope("x"):
        pass
    assert p.items() == [] and p.scope("x") is P.scope("y")  # the shared no-op context
    assert P.Profiler.from_env({"MFQ_PROFILE": "1", "MFQ_PROFILE_FILTER": "attn"}).filter == ("attn",)
    with pytest.raises(ValueError):
        P.Profiler.from_env({"MFQ_PROFILE": "yes"})


def test_engine_profile_names_the_pieces_of_a_step():
    from mfq_b200.engine.llm_engine import LLMEngine
    from mfq_b200.models.llama import LlamaConfig, LlamaModel, LlamaWeights
    cfg = LlamaConfig.tiny()
    engine = LLMEngine(LlamaModel(cfg, LlamaWeights.random_init(cfg, "cpu", seed=1)), max_batch=2, max_seq_len=64, device="cpu")
    items = {it.name: it for it in P.profile_engine(engine, torch.arange(5, 17), decode_tokens=3)}
    assert {"prefill.span", "decode.step", "attn.qkv", "attn.core", "attn.o_proj", "ffn.gate_up", "ffn.down", "head"} <= set(items)
    assert items["decode.step"].calls == 3 and items["prefill.span"].calls == 1
    assert items["attn.qkv"].calls == cfg.num_layers * 4 and items["head"].calls == 4
    assert not P.PROFILER.enabled  # switched back off


def test_profile_command(tmp_path, capsys):
    from mfq_b200.cli import main
    ckpt = tmp_path / "tiny.mfq"
    assert main(["quantize", "synthetic:tiny-moe-128", str(ckpt), "--format", "nint8"]) == 0
    capsys.readouterr()
    assert main(["profile", "--model", str(ckpt), "--device", "cpu", "--prompt-tokens", "12", "--decode-tokens", "2", "--filter", "ffn,decode"]) == 0
    lines = capsys.readouterr().out.strip().splitlines()
    names = [l.split()[1] for l in lines]
    assert all(l.startswith("profile_item name=") for l in lines) and "name=ffn.moe" in names and "name=decode.step" in names
    assert not any("attn" in n for n in names)
