"""Tokenizer, chat template, incremental detokenizer and tool-call parser for the HTTP layer.

``load_tokenizer`` needs ``tokenizer.json`` in the model directory (Hugging Face
``tokenizers``); the chat template comes from ``tokenizer_config.json`` (Jinja) with a
ChatML fallback.  ``IdTokenizer`` is a dependency-free stand-in (token ``i`` renders as
``"<i>"``) used by the simulated engine and by benchmarks that send token-id prompts.

Reference parity: the reference delegates this to the external vllm-server crate;
behaviour pinned by pegainfer-sim/tests/frontend_e2e.rs:174-191,640-665 (tokenizer
files required) and tests/tool_call_roundtrip.rs:1-60 (tool-call extraction).
"""
from __future__ import annotations

import json
import os
import re
from typing import Optional


class IdTokenizer:
    """``"<17><4>"`` <-> ``[17, 4]``; plain text maps to its UTF-8 bytes."""

    eos_token_id = None

    def __init__(self, vocab_size: int = 1 << 30):
        self.vocab_size = vocab_size

    def encode(self, text: str) -> list:
        ids = re.findall(r"<(\d+)>", text)
        if ids and "".join(f"<{i}>" for i in ids) == text:
            return [int(i) % self.vocab_size for i in ids]
        return [b % self.vocab_size for b in text.encode("utf-8")]

    def decode(self, ids) -> str:
        return "".join(f"<{int(i)}>" for i in ids)

    def apply_chat_template(self, messages, tools=None, add_generation_prompt=True) -> list:
        return self.encode(render_chatml(messages, tools, add_generation_prompt))


class HfTokenizer:
    def __init__(self, model_dir: str):
        from tokenizers import Tokenizer

        path = os.path.join(model_dir, "tokenizer.json")
        if not os.path.exists(path):
            raise FileNotFoundError(f"no supported tokenizer file in {model_dir}: expected tokenizer.json")
        self.tok = Tokenizer.from_file(path)
        self.template = None
        self.eos_token_id = None
        cfg_path = os.path.join(model_dir, "tokenizer_config.json")
        if os.path.exists(cfg_path):
            with open(cfg_path) as f:
                cfg = json.load(f)
            self.template = cfg.get("chat_template")
            eos = cfg.get("eos_token")
            if isinstance(eos, dict):
                eos = eos.get("content")
            if eos:
                self.eos_token_id = self.tok.token_to_id(eos)

    def encode(self, text: str) -> list:
        return self.tok.encode(text, add_special_tokens=False).ids

    def decode(self, ids) -> str:
        return self.tok.decode(list(ids), skip_special_tokens=True)

    def apply_chat_template(self, messages, tools=None, add_generation_prompt=True) -> list:
        if self.template:
            try:
                import jinja2

                env = jinja2.Environment()
                text = env.from_string(self.template).render(messages=messages, tools=tools, add_generation_prompt=add_generation_prompt)
                return self.encode(text)
            except Exception:
                pass
        return self.encode(render_chatml(messages, tools, add_generation_prompt))


def render_chatml(messages, tools=None, add_generation_prompt=True) -> str:
    parts = []
    if tools:
        parts.append("<|im_start|>system\n# Tools\n" + "\n".join(json.dumps(t) for t in tools) + "<|im_end|>\n")
    for m in messages:
        content = m.get("content")
        if isinstance(content, list):
            content = "".join(p.get("text", "") for p in content if isinstance(p, dict))
        parts.append(f"<|im_start|>{m.get('role', 'user')}\n{content or ''}<|im_end|>\n")
    if add_generation_prompt:
        parts.append("<|im_start|>assistant\n")
    return "".join(parts)


def load_tokenizer(model_dir: Optional[str], vocab_size: int = 1 << 30):
    if model_dir is None:
        return IdTokenizer(vocab_size)
    return HfTokenizer(model_dir)


class IncrementalDetokenizer:
    """Turns a growing id list into text deltas; holds back an incomplete UTF-8 tail."""

    def __init__(self, tokenizer):
        self.tok = tokenizer
        self.ids: list = []
        self.emitted = ""

    def push(self, new_ids) -> str:
        self.ids.extend(new_ids)
        text = self.tok.decode(self.ids)
        if text.endswith("\ufffd"):
            return ""
        delta = text[len(self.emitted) :]
        self.emitted = text
        return delta


_TOOL_RE = re.compile(r"<tool_call>\s*(\{.*?\})\s*</tool_call>", re.S)


def extract_tool_calls(text: str):
    """Split model text into (plain content, [OpenAI tool_call dicts])."""
    calls = []
    for i, m in enumerate(_TOOL_RE.finditer(text)):
        try:
            obj = json.loads(m.group(1))
        except json.JSONDecodeError:
            continue
        args = obj.get("arguments", obj.get("parameters", {}))
        calls.append({"id": f"call_{i}", "type": "function", "function": {"name": obj.get("name", ""), "arguments": args if isinstance(args, str) else json.dumps(args)}})
    content = _TOOL_RE.sub("", text).strip() if calls else text
    return content, calls
