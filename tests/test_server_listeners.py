"""One application on two ports (OpenAI-facing and Anthropic-facing listeners), over real sockets on the loopback."""

import requests

from mfq_b200.server import ModelService, create_app
from mfq_b200.server.listen import Listeners
from mfq_b200.server.tokenizer import ByteTokenizer
from test_server import EchoBackend


def test_two_listeners_serve_the_same_model():
    service = ModelService(max_queue=2, queue_timeout=5.0)
    service.add_model("echo", EchoBackend(max_batch=2), ByteTokenizer())
    # two ephemeral ports: ask the OS for them by binding port 0 twice (distinct Config objects)
    import uvicorn
    app = create_app(service)
    ls = Listeners(app, "127.0.0.1", [0])
    ls.servers.append(uvicorn.Server(uvicorn.Config(app, host="127.0.0.1", port=0, log_level="warning")))
    ls.start()
    try:
        a, b = ls.ports()[:2]
        assert a != b
        r = requests.post(f"http://127.0.0.1:{a}/v1/chat/completions", timeout=30,
                          json={"model": "echo", "messages": [{"role": "user", "content": "hi"}], "max_tokens": 8})
        assert r.status_code == 200 and r.json()["choices"][0]["message"]["content"] == "ok!"
        r = requests.post(f"http://127.0.0.1:{b}/v1/messages", timeout=30,
                          json={"model": "echo", "max_tokens": 8, "messages": [{"role": "user", "content": "hi"}]})
        assert r.status_code == 200 and r.json()["content"][0]["text"] == "ok!"
        assert requests.get(f"http://127.0.0.1:{b}/health", timeout=10).json()["model"] == "echo"
    finally:
        ls.stop()
        service.shutdown()
    assert not any(t.is_alive() for t in ls.threads)
