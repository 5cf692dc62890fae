"""Model benchmark driver: the matrix over the stdio runtime on a tiny CPU checkpoint, and the report renderers."""

import json

from mfq_b200.cli import main
from mfq_b200.evaluation import model_bench as mb


def test_matrix_over_the_stdio_runtime_and_reports(tmp_path, capsys):
    ckpt = tmp_path / "tiny.mfq"
    assert main(["quantize", "synthetic:tiny-moe-128", str(ckpt), "--format", "nint8"]) == 0
    capsys.readouterr()
    out, page = tmp_path / "r.json", tmp_path / "r.html"
    assert main(["bench-model", "--model", str(ckpt), "--device", "cpu", "--prompt-tokens", "8,24", "--new-tokens", "4",
                 "--concurrency", "1,2", "--repeats", "2", "--warmup", "1", "--output", str(out), "--html", str(page)]) == 0
    md = capsys.readouterr().out
    report = json.loads(out.read_text())
    assert report["format"] == "mfq.model-bench.v1" and report["models"] == ["tiny"] and len(report["rows"]) == 4
    for r in report["rows"]:
        assert r["ttft_ms"] > 0 and r["prefill_tps"] > 0 and r["aggregate_tps"] > 0
        assert 1 <= r["completion_tokens"] <= 4 * r["concurrency"]
    assert [(r["prompt_tokens"], r["concurrency"]) for r in report["rows"]] == [(8, 1), (8, 2), (24, 1), (24, 2)]
    assert md.count("\n| ") >= 5 and "prefill tok/s" in md
    text = page.read_text()
    assert text.startswith("<!doctype html>") and text.count("<tr>") == 5
    assert main(["bench-model", "--render", str(out)]) == 0
    assert "TTFT ms" in capsys.readouterr().out


def test_report_validation():
    good = {"format": "mfq.model-bench.v1", "rows": [{"prompt_tokens": 8, "concurrency": 2, "new_tokens": 4, "ttft_ms": 1.0,
                                                      "prefill_tps": 10.0, "decode_tps": 5.0, "aggregate_tps": 5.0, "completion_tokens": 8}]}
    assert mb.validate_report(good) == []
    bad = {"format": "x", "rows": [dict(good["rows"][0], ttft_ms=0.0, completion_tokens=9), good["rows"][0], good["rows"][0]]}
    msgs = " | ".join(mb.validate_report(bad))
    assert "unknown format" in msgs and "ttft_ms" in msgs and "9 completion tokens for 8" in msgs and "appears twice" in msgs
    assert mb.validate_report({"format": "mfq.model-bench.v1", "rows": []}) == ["no rows"]


def test_renderers_escape_and_scale():
    report = {"label": "<x>", "command": ["a", "<b>"], "rows": [
        {"prompt_tokens": 1, "concurrency": 1, "new_tokens": 2, "ttft_ms": 1.0, "prefill_tps": 10.0, "decode_tps": 5.0, "aggregate_tps": 5.0},
        {"prompt_tokens": 1, "concurrency": 2, "new_tokens": 2, "ttft_ms": 2.0, "prefill_tps": 10.0, "decode_tps": 4.0, "aggregate_tps": 10.0}]}
    page = mb.render_html(report)
    assert "&lt;x&gt;" in page and "&lt;b&gt;" in page and "width:50.0%" in page and "width:100.0%" in page
    assert "| 1 | 2 | 2 | 2.0 | 10 | 4.0 | 10.0 |" in mb.render_markdown(report)
