"""Tokenizer adapters for serving.

A checkpoint may embed a Hugging Face ``tokenizer.json`` (asset ``hf/tokenizer.json``) and a Jinja chat template
(``hf/chat_template.jinja``); both are used when present (``tokenizers`` / ``jinja2`` are optional imports).  Without
them -- e.g. the random-init benchmark models -- a reversible byte-level fallback keeps the HTTP surface usable.
The reference renders chat templates and tokenizes inside its native worker (``cpp_runtime/components/tokenizer``).
"""

from __future__ import annotations

import json


class ByteTokenizer:
    """UTF-8 bytes as token ids (offset by 3 for specials); ids beyond that range decode to '?'."""

    bos_id, eos_id, pad_id = 1, 2, 0

    def __init__(self, vocab_size: int = 259) -> None:
        self.vocab_size = max(vocab_size, 259)

    def encode(self, text: str) -> list[int]:
        return [b + 3 for b in text.encode("utf-8")]

    def decode(self, ids) -> str:
        data = bytes((i - 3) for i in ids if 3 <= i < 259)
        text = data.decode("utf-8", errors="ignore")
        return text + "?" * sum(1 for i in ids if i >= 259)

    def token_bytes(self, vocab_size: int | None = None) -> list[bytes]:
        """Bytes each token id adds to the text (empty for specials and unused ids); for token constraints."""
        n = vocab_size or self.vocab_size
        return [bytes([i - 3]) if 3 <= i < 259 else b"" for i in range(n)]

    def apply_chat_template(self, messages: list[dict], add_generation_prompt: bool = True, **_template_vars) -> str:
        parts = [f"<|{m['role']}|>\n{_content_text(m.get('content'))}\n" for m in messages]
        if add_generation_prompt:
            parts.append("<|assistant|>\n")
        return "".join(parts)

    @property
    def stop_ids(self) -> tuple[int, ...]:
        return (self.eos_id,)


class HfTokenizer:
    def __init__(self, tokenizer_json: bytes, chat_template: str | None = None, eos_token: str | None = None) -> None:
        from tokenizers import Tokenizer
        self.tk = Tokenizer.from_str(tokenizer_json.decode("utf-8"))
        self.vocab_size = self.tk.get_vocab_size()
        self.chat_template = chat_template
        self.eos_id = self.tk.token_to_id(eos_token) if eos_token else None

    def encode(self, text: str) -> list[int]:
        return self.tk.encode(text, add_special_tokens=False).ids

    def decode(self, ids) -> str:
        return self.tk.decode(list(ids), skip_special_tokens=True)

    def token_bytes(self, vocab_size: int | None = None) -> list[bytes]:
        """Bytes each token id adds to the text; empty for special / added control tokens and ids past the vocabulary.
        Byte-level BPE vocabularies are mapped back through the GPT-2 byte alphabet; sentencepiece-style ones through
        the ``\u2581`` space marker and ``<0xNN>`` byte tokens; a piece that cannot be recovered exactly becomes 0xFF
        placeholders (legal inside strings only)."""
        n = vocab_size or self.vocab_size
        spec = json.loads(self.tk.to_str())
        special = {t["id"] for t in spec.get("added_tokens", []) if t.get("special")}
        byte_level = "ByteLevel" in json.dumps(spec.get("decoder") or {}) or "ByteLevel" in json.dumps(spec.get("pre_tokenizer") or {})
        alphabet = _gpt2_byte_alphabet() if byte_level else None
        out = []
        for i in range(n):
            piece = self.tk.id_to_token(i) if i not in special else None
            if piece is None:
                out.append(b"")
            elif alphabet is not None:
                try:
                    out.append(bytes(alphabet[ch] for ch in piece))
                except KeyError:  # an added plain-text token
                    out.append(piece.encode("utf-8"))
            elif len(piece) == 6 and piece.startswith("<0x") and piece.endswith(">"):
                out.append(bytes([int(piece[3:5], 16)]))
            else:
                out.append(piece.replace("\u2581", " ").encode("utf-8"))
        return out

    def apply_chat_template(self, messages: list[dict], add_generation_prompt: bool = True, **template_vars) -> str:
        """``template_vars`` reach the Jinja template as variables (``enable_thinking``, ``tools`` ...)."""
        if self.chat_template:
            import jinja2
            env = jinja2.Environment(trim_blocks=True, lstrip_blocks=True)
            return env.from_string(self.chat_template).render(messages=messages, add_generation_prompt=add_generation_prompt,
                                                              **template_vars)
        return ByteTokenizer.apply_chat_template(self, messages, add_generation_prompt)  # type: ignore[arg-type]

    @property
    def stop_ids(self) -> tuple[int, ...]:
        return (self.eos_id,) if self.eos_id is not None else ()


def _gpt2_byte_alphabet() -> dict[str, int]:
    """Printable stand-in character -> byte, as byte-level BPE vocabularies spell their tokens."""
    keep = list(range(ord("!"), ord("~") + 1)) + list(range(0xA1, 0xAD)) + list(range(0xAE, 0x100))
    table, extra = {}, 0
    for b in range(256):
        if b in keep:
            table[chr(b)] = b
        else:
            table[chr(256 + extra)] = b
            extra += 1
    return table


def _content_text(content) -> str:
    """OpenAI/Anthropic message content: a string, or a list of typed parts (text parts are concatenated)."""
    if content is None:
        return ""
    if isinstance(content, str):
        return content
    return "".join(p.get("text", "") for p in content if isinstance(p, dict) and p.get("type") in ("text", "input_text"))


def tokenizer_from_assets(assets: dict[str, bytes], vocab_size: int):
    tj = assets.get("hf/tokenizer.json")
    if tj:
        try:
            template = assets.get("hf/chat_template.jinja")
            cfg = json.loads(assets.get("hf/tokenizer_config.json", b"{}"))
            eos = cfg.get("eos_token") if isinstance(cfg.get("eos_token"), str) else None
            return HfTokenizer(tj, template.decode("utf-8") if template else cfg.get("chat_template"), eos)
        except Exception:  # missing optional dependency or malformed asset: stay usable
            pass
    return ByteTokenizer(vocab_size)
