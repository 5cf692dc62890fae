"""Tool calls through the HTTP surface: tools reach the prompt, <tool_call> blocks come back as structured calls."""

import json

import pytest
from fastapi.testclient import TestClient

from mfq_b200.server import ModelService, create_app, tools
from mfq_b200.server.tokenizer import ByteTokenizer
from test_scheduler import FakeBackend

CALL = 'Let me check.<tool_call>{"name": "get_weather", "arguments": {"city": "Oslo"}}</tool_call>'


class ScriptedBackend(FakeBackend):
    """Emits a fixed text (byte tokenizer ids are byte + 3), remembers the prompt it was given."""
    text = CALL

    def prefill(self, row, tokens, params):
        super().prefill(row, tokens, params)
        self.last_prompt = bytes(t - 3 for t in tokens if t >= 3).decode("utf-8", errors="replace")
        self.script = {row: [b + 3 for b in self.text.encode()] + [2]}
        return self.script[row].pop(0)

    def decode(self, rows):
        return {r: (self.script[r].pop(0) if self.script[r] else 2) for r in rows}


def test_extract_and_prompt_helpers():
    text, calls = tools.extract(CALL)
    assert text == "Let me check." and calls[0]["name"] == "get_weather" and calls[0]["arguments"] == {"city": "Oslo"}
    broken = "<tool_call>{not json}</tool_call>"
    assert tools.extract(broken) == (broken, [])
    spec = tools.normalise([{"type": "function", "function": {"name": "f", "parameters": {"type": "object"}}},
                            {"name": "g", "input_schema": {"type": "object"}}])
    assert [t["name"] for t in spec] == ["f", "g"]
    msgs = tools.with_tools([{"role": "user", "content": "hi"}, {"role": "tool", "content": "42"}], spec)
    assert msgs[0]["role"] == "system" and '"name": "f"' in msgs[0]["content"] and "<tool_response>42" in msgs[2]["content"]


@pytest.fixture()
def client():
    service = ModelService(max_queue=2, queue_timeout=5.0)
    backend = ScriptedBackend(max_batch=2)
    service.add_model("m", backend, ByteTokenizer())
    with TestClient(create_app(service)) as c:
        yield c, backend
    service.shutdown()


def test_openai_and_anthropic_tool_calls(client):
    c, backend = client
    spec = [{"type": "function", "function": {"name": "get_weather", "description": "weather", "parameters": {"type": "object"}}}]
    r = c.post("/v1/chat/completions", json={"model": "m", "messages": [{"role": "user", "content": "weather?"}], "tools": spec,
                                             "max_tokens": 200})
    choice = r.json()["choices"][0]
    assert choice["finish_reason"] == "tool_calls" and choice["message"]["content"] == "Let me check."
    call = choice["message"]["tool_calls"][0]
    assert call["function"]["name"] == "get_weather" and json.loads(call["function"]["arguments"]) == {"city": "Oslo"}
    assert "get_weather" in backend.last_prompt and "<tool_call>" in backend.last_prompt  # the tool list and the syntax were shown
    # without tools in the request the text is returned as it is
    r = c.post("/v1/chat/completions", json={"model": "m", "messages": [{"role": "user", "content": "x"}], "max_tokens": 200})
    assert "<tool_call>" in r.json()["choices"][0]["message"]["content"]
    r = c.post("/v1/messages", json={"model": "m", "max_tokens": 200, "messages": [{"role": "user", "content": "weather?"}],
                                     "tools": [{"name": "get_weather", "input_schema": {"type": "object"}}]})
    body = r.json()
    assert body["stop_reason"] == "tool_use" and body["content"][0] == {"type": "text", "text": "Let me check."}
    assert body["content"][1]["type"] == "tool_use" and body["content"][1]["input"] == {"city": "Oslo"}


def test_reasoning_block_is_split_from_the_answer(client):
    c, backend = client
    assert tools.split_reasoning("<think>a\nb</think>\n\nfinal") == ("a\nb", "final")
    assert tools.split_reasoning("plain") == (None, "plain") and tools.split_reasoning("<think>cut off") == ("cut off", "")
    backend.text = "<think>the user greets me</think>Hello!"
    r = c.post("/v1/chat/completions", json={"model": "m", "messages": [{"role": "user", "content": "hi"}], "max_tokens": 200})
    msg = r.json()["choices"][0]["message"]
    assert msg["content"] == "Hello!" and msg["reasoning_content"] == "the user greets me"


def test_enable_thinking_reaches_the_chat_template():
    import json as _json
    from mfq_b200.server.tokenizer import HfTokenizer
    spec = {"version": "1.0", "truncation": None, "padding": None, "added_tokens": [], "normalizer": None, "pre_tokenizer": None,
            "post_processor": None, "decoder": None,
            "model": {"type": "WordLevel", "vocab": {"<unk>": 0, "a": 1}, "unk_token": "<unk>"}}
    template = "{% for m in messages %}{{ m.content }}{% endfor %}{% if enable_thinking is defined and not enable_thinking %}<think></think>{% endif %}"
    tok = HfTokenizer(_json.dumps(spec).encode(), template)
    msgs = [{"role": "user", "content": "a"}]
    assert tok.apply_chat_template(msgs) == "a" and tok.apply_chat_template(msgs, enable_thinking=True) == "a"
    assert tok.apply_chat_template(msgs, enable_thinking=False) == "a<think></think>"
