"""Runtime configuration: typed record, strict MFQ_* parsing, trace lines."""

import json

import pytest

from mfq_b200 import config as C


def test_defaults_overrides_and_strict_values(capsys):
    d = C.RuntimeConfig.from_env({})
    assert d.gemv and d.pdl and d.cuda_graphs and d.gemm_stages == 0 and d.prefill_chunk == 8192 and d.trace == ()
    c = C.RuntimeConfig.from_env({"MFQ_GEMV": "0", "MFQ_GEMM_STAGES": "4", "MFQ_PREFILL_CHUNK": "2048", "MFQ_TRACE": "scheduler,graph",
                                  "MFQ_PROFILE": "1", "MFQ_PROFILE_FILTER": "attn", "PATH": "/bin"})
    assert not c.gemv and c.gemm_stages == 4 and c.prefill_chunk == 2048 and c.traces("graph") and not c.traces("prefix")
    assert c.profile and c.profile_filter == "attn"
    for bad in ({"MFQ_GEMV": "off"}, {"MFQ_GEMM_STAGES": "5"}, {"MFQ_PREFILL_CHUNK": "0"}, {"MFQ_TRACE": "everything"},
                {"MFQ_NATIVE_THREADS": "many"}):
        with pytest.raises(ValueError, match=next(iter(bad))):
            C.RuntimeConfig.from_env(bad)
    C.RuntimeConfig.from_env({"MFQ_GEMW": "1"})  # a misspelt name is reported, not fatal
    assert "MFQ_GEMW" in capsys.readouterr().err
    assert C.RuntimeConfig.from_env({"MFQ_TRACE": "all"}).traces("spmd")


def test_describe_and_command(capsys, monkeypatch):
    rows = C.RuntimeConfig().describe()
    assert {r["variable"] for r in rows} >= {"MFQ_GEMV", "MFQ_PDL", "MFQ_GEMM_STAGES", "MFQ_CUDA_GRAPHS", "MFQ_TRACE"}
    from mfq_b200.cli import main
    monkeypatch.setenv("MFQ_PREFILL_CHUNK", "1024")
    assert main(["config", "--json"]) == 0
    got = {r["variable"]: r for r in json.loads(capsys.readouterr().out)}
    assert got["MFQ_PREFILL_CHUNK"]["value"] == 1024 and got["MFQ_PREFILL_CHUNK"]["default"] == 8192
    assert main(["config"]) == 0 and "(set)" in capsys.readouterr().out


def test_trace_lines_follow_the_scheduler(capsys):
    from mfq_b200.engine.scheduler import ContinuousBatchScheduler, Request, SamplingParams
    from test_scheduler import FakeBackend
    try:
        C.reload({"MFQ_TRACE": "scheduler"})
        sched = ContinuousBatchScheduler(FakeBackend(max_batch=2), max_queue=4)
        sched.submit(Request([1, 2, 3], SamplingParams(max_tokens=2)))
        for _ in range(10):
            if not sched.step() and sched.idle:
                break
        err = capsys.readouterr().err
        assert "trace topic=scheduler event=admit" in err and "event=finish" in err and "row=0" in err
        C.reload({})
        C.trace("scheduler", "admit", row=1)
        assert capsys.readouterr().err == ""
    finally:
        C.reload({})
