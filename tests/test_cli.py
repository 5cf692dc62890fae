"""`mfq` command line on a synthetic tiny MoE: quantize (mixed experts), inspect, eval kl, and loading into the engine."""

import json

import torch

from mfq_b200.cli import main


def test_quantize_inspect_eval_and_load(tmp_path, capsys):
    base, mixed = tmp_path / "base.mfq", tmp_path / "mixed.mfq"
    assert main(["quantize", "synthetic:tiny-moe-128", str(base), "--full-precision"]) == 0
    assert main(["quantize", "synthetic:tiny-moe-128", str(mixed), "--format", "nint4", "--random-expert-mix", "NINT4,NVQ3,MXFP4"]) == 0
    capsys.readouterr()
    assert main(["inspect", str(mixed)]) == 0
    info = json.loads(capsys.readouterr().out)
    assert info["arch"] == "mfq_b200_decoder" and "MFE" in info["bytes_by_dtype"] and "NINT" in info["bytes_by_dtype"]
    assert info["extra"]["quantization"]["random_expert_mix"] == ["NINT4", "NVQ3", "MXFP4"]
    assert mixed.stat().st_size < 0.5 * base.stat().st_size
    assert main(["eval", "kl", "--model", str(mixed), "--base", str(base), "--chunks", "2", "--ctx", "64"]) == 0
    line = capsys.readouterr().out.strip()
    assert line.startswith("kld=") and "same_top=" in line
    assert float(line.split()[0].split("=")[1]) < 0.01
    assert main(["quantize", "synthetic:tiny-moe-128", str(mixed), "--dry-run"]) == 0
    # re-quantizing an .mfq source and loading the result into the serving engine (CPU path)
    again = tmp_path / "again.mfq"
    assert main(["quantize", str(base), str(again), "--format", "nint8"]) == 0
    from mfq_b200.checkpoint import load_engine
    engine, tok, cfg = load_engine(again, "cpu", max_batch=2, max_seq_len=64)
    out = engine.generate([torch.tensor(tok.encode("hello"))], 4)
    assert out.tokens.shape == (1, 4) and cfg.num_experts == 8


def test_preset_imatrix_alphaq_flow(tmp_path, capsys):
    """quantize --preset (role-based widths), calibrate imatrix -> quantize --imatrix, calibrate alphaq."""
    import json

    from mfq_b200 import cli, formats as F
    out = tmp_path / "p.mfq"
    assert cli.main(["quantize", "synthetic:tiny-moe", str(out), "--preset", "S3-M"]) == 0
    with F.open_mfq(out) as st:
        widths = {n: int(st[n].spec.bits) for n in st if st.dtype(n) == "NINT"}
        assert st.header.extra["quantization"]["preset"] == "S3-M"
    assert widths["model.output.weight"] == 6 and widths["model.block.0.attention.value.weight"] == 5
    assert widths["model.block.0.attention.query.weight"] == 3 and widths["model.block.0.attention.output.weight"] == 4
    im = tmp_path / "im.npz"
    assert cli.main(["calibrate", "imatrix", "synthetic:tiny-moe", "--output", str(im), "--chunks", "2", "--ctx", "32"]) == 0
    assert cli.main(["quantize", "synthetic:tiny-moe", str(tmp_path / "q.mfq"), "--bits", "4", "--imatrix", str(im)]) == 0
    aq = tmp_path / "aq.json"
    assert cli.main(["calibrate", "alphaq", "synthetic:tiny-moe", "--output", str(aq), "--target-bpw", "4.0"]) == 0
    doc = json.loads(aq.read_text())
    assert doc["format"] == "mfq.alphaq-allocation.v1" and len(doc["tensors"]) > 10
    capsys.readouterr()


def test_diagnose_runs_the_format_checks_on_cpu(capsys):
    import json
    from mfq_b200.cli import main
    assert main(["diagnose", "--check", "nint", "--check", "container", "--check", "fp8-block"]) == 0
    report = json.loads(capsys.readouterr().out)
    assert report["ok"] and set(report["checks"]) == {"nint", "container", "fp8-block"}
    assert report["checks"]["nint"]["snr_db"] > 18
    assert main(["diagnose", "--check", "tp-linear", "--check", "ep-moe", "--check", "continuous-batching", "--check", "json-constraint"]) == 0
    report = json.loads(capsys.readouterr().out)
    assert report["ok"] and report["checks"]["ep-moe"]["ranks_identical"] and report["checks"]["continuous-batching"]["identical"] == 5
    assert [c["world"] for c in report["checks"]["tp-linear"]["cases"]] == [2, 4]


def test_wt2_reference_and_eval_against_it(tmp_path, capsys):
    """Baseline checkpoint -> reference-logits file -> `eval kl --base <file>`: the baseline scores ~0 KLD against its own
    file, a 3-bit quantization scores worse."""
    import json
    from mfq_b200.cli import main
    base, q3, ref = tmp_path / "base.mfq", tmp_path / "q3.mfq", tmp_path / "base._logit3_"
    assert main(["quantize", "synthetic:tiny-moe", str(base), "--full-precision"]) == 0
    assert main(["quantize", "synthetic:tiny-moe", str(q3), "--bits", "3"]) == 0
    capsys.readouterr()
    assert main(["wt2-reference", "--model", str(base), "--output", str(ref), "--chunks", "2", "--ctx", "32"]) == 0
    info = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert info["chunks"] == 2 and ref.exists() and info["baseline_ppl"] > 1
    assert main(["eval", "kl", "--model", str(base), "--base", str(ref)]) == 0
    own = dict(kv.split("=") for kv in capsys.readouterr().out.split())
    assert main(["eval", "kl", "--model", str(q3), "--base", str(ref)]) == 0
    quant = dict(kv.split("=") for kv in capsys.readouterr().out.split())
    assert float(own["kld"]) < 1e-3 and float(own["same_top"]) > 0.97
    assert float(quant["kld"]) > float(own["kld"])


def test_optimize_layout_transcodes_to_the_runtime_format(tmp_path, capsys):
    import json
    from mfq_b200 import formats as F
    from mfq_b200.cli import main
    src, dst = tmp_path / "q4.mfq", tmp_path / "native.mfq"
    # groups of 32 divide the 256-wide rows, which is what the 4-bit GEMM needs to take a tensor as it is
    assert main(["quantize", "synthetic:tiny-moe-128", str(src), "--bits", "4", "--groupsize", "32",
                 "--random-expert-mix", "NINT4,NVQ3,MXFP4"]) == 0
    capsys.readouterr()
    assert main(["optimize-layout", "--input", str(src), "--output", str(dst), "--keep-4bit"]) == 0
    info = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert info["transcoded"] > 0 and info["kept_4bit"] > 0
    with F.open_mfq(dst) as store:
        assert store.header.extra["layout"]["dense"] == "FP8-128SQ"
        dtypes = {n: store.dtype(n) for n in store if not n.startswith("__mfq_asset__/")}
        assert "model_graph.json" in store.assets()
    assert dtypes["model.block.0.attention.query.weight"].startswith("NINT")       # kept as 4-bit
    assert dtypes["model.block.0.mlp.experts.gate.weight"] == "MFE"                 # experts re-pooled as FP8
    # the optimized file serves the same model (KLD against the 4-bit source is tiny: FP8 on top of the 4-bit values)
    assert main(["eval", "kl", "--model", str(dst), "--base", str(src), "--chunks", "1", "--ctx", "32"]) == 0
    kld = float(capsys.readouterr().out.split("kld=")[1].split()[0])
    assert kld < 0.02
    import pytest
    with pytest.raises(SystemExit):  # an existing output needs --overwrite
        main(["optimize-layout", "--input", str(src), "--output", str(dst)])


def test_sharded_output_opens_as_one_checkpoint(tmp_path, capsys):
    import json
    from mfq_b200 import formats as F
    from mfq_b200.cli import main
    whole, stem = tmp_path / "whole.mfq", tmp_path / "parts.mfq"
    assert main(["quantize", "synthetic:tiny-moe", str(whole), "--bits", "4"]) == 0
    capsys.readouterr()
    assert main(["quantize", "synthetic:tiny-moe", str(stem), "--bits", "4", "--shard-size-gb", "0.0003"]) == 0
    info = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert info["shards"] >= 3 and info["output"].endswith("-00001-of-%05d.mfq" % info["shards"])
    with F.open_mfq(whole) as a, F.open_mfq(info["output"]) as b:
        assert sorted(a) == sorted(b) and a.assets()["model_config.json"] == b.assets()["model_config.json"]
        n = "model.block.1.attention.output.weight"
        assert (F.dequantize(a[n]) == F.dequantize(b[n])).all()
    # a sharded checkpoint is a valid input of the other commands
    assert main(["inspect", info["output"]]) == 0
