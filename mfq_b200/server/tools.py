"""Tool calls: how tool definitions reach the prompt and how calls come back out of generated text.

Prompt side: the request's ``tools`` are handed to the chat template (``tools=`` like Hugging Face templates expect);
templates that ignore them get a system block that lists the tools as JSON and states the call syntax.  Output side:
``<tool_call>{"name": ..., "arguments": {...}}</tool_call>`` blocks (the Qwen / Hermes convention the reference's
XML tool-call protocol uses, ``mfq/server/protocol``) are cut out of the text and returned as OpenAI ``tool_calls`` or
Anthropic ``tool_use`` blocks.  A block that is not valid JSON stays in the text untouched.
"""

from __future__ import annotations

import json
import re
import uuid

_CALL = re.compile(r"<tool_call>\s*(\{.*?\})\s*</tool_call>", re.S)
SYNTAX = ('To call a tool, answer with <tool_call>{"name": <tool name>, "arguments": <arguments as a JSON object>}</tool_call> '
          "and nothing after it.")


def normalise(tools: list[dict] | None) -> list[dict]:
    """OpenAI (``{"type": "function", "function": {...}}``) and Anthropic (``{"name", "description", "input_schema"}``)
    tool definitions -> ``{"name", "description", "parameters"}``."""
    out = []
    for t in tools or []:
        f = t.get("function", t)
        if "name" in f:
            out.append({"name": f["name"], "description": f.get("description", ""),
                        "parameters": f.get("parameters") or f.get("input_schema") or {"type": "object", "properties": {}}})
    return out


def system_block(tools: list[dict]) -> str:
    return "You may call these tools:\n" + "\n".join(json.dumps(t, sort_keys=True) for t in tools) + "\n" + SYNTAX


def with_tools(messages: list[dict], tools: list[dict]) -> list[dict]:
    """Messages with the tool list folded into the (first) system message, for templates without tool support; tool
    results (role ``tool``) become user-visible text."""
    if not tools:
        return messages
    block = system_block(tools)
    out, placed = [], False
    for m in messages:
        if m.get("role") == "system" and not placed:
            out.append({**m, "content": f"{m.get('content') or ''}\n\n{block}".strip()})
            placed = True
        elif m.get("role") == "tool":
            out.append({"role": "user", "content": f"<tool_response>{m.get('content')}</tool_response>"})
        elif m.get("role") == "assistant" and m.get("tool_calls"):
            calls = "".join(f"<tool_call>{json.dumps({'name': c['function']['name'], 'arguments': json.loads(c['function'].get('arguments') or '{}')})}</tool_call>"
                            for c in m["tool_calls"])
            out.append({"role": "assistant", "content": f"{m.get('content') or ''}{calls}"})
        else:
            out.append(m)
    if not placed:
        out.insert(0, {"role": "system", "content": block})
    return out


def extract(text: str) -> tuple[str, list[dict]]:
    """-> (text without the call blocks, calls as ``{"id", "name", "arguments"}`` with ``arguments`` a dict)."""
    calls = []

    def take(match):
        try:
            obj = json.loads(match.group(1))
            name, args = obj["name"], obj.get("arguments", {})
            if isinstance(args, str):
                args = json.loads(args)
            if not isinstance(name, str) or not isinstance(args, dict):
                raise ValueError
        except (ValueError, KeyError, TypeError):
            return match.group(0)
        calls.append({"id": f"call_{uuid.uuid4().hex[:24]}", "name": name, "arguments": args})
        return ""

    rest = _CALL.sub(take, text)
    return (rest.strip() if calls else text), calls


def openai_calls(calls: list[dict]) -> list[dict]:
    return [{"id": c["id"], "type": "function", "function": {"name": c["name"], "arguments": json.dumps(c["arguments"])}} for c in calls]


def anthropic_blocks(text: str, calls: list[dict]) -> list[dict]:
    blocks = [{"type": "text", "text": text}] if text or not calls else []
    return blocks + [{"type": "tool_use", "id": c["id"].replace("call_", "toolu_"), "name": c["name"], "input": c["arguments"]} for c in calls]


_THINK = re.compile(r"^\s*<think>(.*?)</think>\s*", re.S)


def split_reasoning(text: str) -> tuple[str | None, str]:
    """A leading ``<think>...</think>`` block (reasoning models) -> (reasoning, remaining answer); an unterminated block
    (generation stopped while thinking) is all reasoning."""
    m = _THINK.match(text)
    if m:
        return m.group(1).strip(), text[m.end():]
    stripped = text.lstrip()
    if stripped.startswith("<think>"):
        return stripped[len("<think>"):].strip(), ""
    return None, text
