"""Idle models are unloaded after --runtime-idle-timeout and come back on demand through the loader."""

import time

from mfq_b200.engine.scheduler import SamplingParams
from mfq_b200.server import ModelService
from mfq_b200.server.tokenizer import ByteTokenizer
from test_server import EchoBackend


def test_idle_model_is_unloaded_and_reloaded():
    loads = []

    def loader(name):
        loads.append(name)
        return EchoBackend(max_batch=2), ByteTokenizer()

    service = ModelService(max_queue=4, queue_timeout=5.0, loader=loader, idle_timeout=0.3)
    try:
        lm = service.load("echo")
        _req, events = service.submit(lm, [5, 6, 7], SamplingParams(max_tokens=4, stop_token_ids=(2,)))
        while events.get(True, 10).kind == "token":
            pass
        assert "echo" in service.models
        deadline = time.time() + 10
        while "echo" in service.models and time.time() < deadline:
            time.sleep(0.05)
        assert "echo" not in service.models
        again = service.resolve("echo")
        assert again is not lm and loads == ["echo", "echo"]
    finally:
        service.shutdown()


def test_without_a_loader_nothing_is_unloaded():
    service = ModelService(idle_timeout=0.05)
    try:
        service.add_model("echo", EchoBackend(max_batch=1), ByteTokenizer())
        time.sleep(0.4)
        assert "echo" in service.models
    finally:
        service.shutdown()
