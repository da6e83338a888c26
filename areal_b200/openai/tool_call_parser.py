"""Extraction of tool calls and reasoning from generated text (reference:
``areal/experimental/openai/tool_call_parser.py``). Supports the Qwen / Hermes convention
``<tool_call>{"name": ..., "arguments": {...}}</tool_call>`` and ``<think>...</think>``."""
from __future__ import annotations

import json
import re
from typing import Optional

from .types import FunctionCall, ToolCall

_TOOL_RE = re.compile(r"<tool_call>\s*(\{.*?\})\s*</tool_call>", re.S)
_THINK_RE = re.compile(r"<think>(.*?)</think>", re.S)


def parse_tool_calls(text: str, tools: Optional[list[dict]] = None) -> tuple[str, list[ToolCall]]:
    """Returns (text without the tool-call blocks, parsed calls). Blocks that are not valid
    JSON or name an unknown tool stay in the text."""
    known = None
    if tools:
        known = {t.get("function", t).get("name") for t in tools}
    calls: list[ToolCall] = []

    def repl(m: re.Match) -> str:
        try:
            obj = json.loads(m.group(1))
        except json.JSONDecodeError:
            return m.group(0)
        name = obj.get("name")
        if not isinstance(name, str) or (known is not None and name not in known):
            return m.group(0)
        args = obj.get("arguments", obj.get("parameters", {}))
        calls.append(ToolCall(function=FunctionCall(name=name, arguments=args if isinstance(args, str) else json.dumps(args))))
        return ""
    rest = _TOOL_RE.sub(repl, text)
    return rest.strip() if calls else text, calls


def split_reasoning(text: str) -> tuple[Optional[str], str]:
    m = _THINK_RE.search(text)
    if not m:
        return None, text
    return m.group(1).strip(), (text[: m.start()] + text[m.end():]).strip()
