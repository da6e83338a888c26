"""Extraction of tool calls and reasoning from generated text (reference:
``areal/experimental/openai/tool_call_parser.py``). Formats (``parser`` argument):

* ``qwen25`` / ``hermes``: ``<tool_call>{"name": ..., "arguments": {...}}</tool_call>``;
* ``qwen3_coder``: ``<tool_call><function=NAME><parameter=KEY>VALUE</parameter>...</function></tool_call>``
  with values coerced to the JSON types of the tool's schema (reference :106-255);
* ``json`` / ``llama3_json``: the whole message (or a fenced block) is one JSON object or a list of
  objects ``{"name": ..., "arguments" | "parameters": {...}}``;
* ``auto``: whichever of the above matches.

``<think>...</think>`` blocks are split off by :func:`split_reasoning`."""
from __future__ import annotations

import json
import re
from typing import Optional

from .types import FunctionCall, ToolCall

_TOOL_RE = re.compile(r"<tool_call>\s*(\{.*?\})\s*</tool_call>", re.S)
_THINK_RE = re.compile(r"<think>(.*?)</think>", re.S)


_CODER_RE = re.compile(r"<tool_call>\s*<function=([^>\s]+)>(.*?)</function>\s*</tool_call>", re.S)
_PARAM_RE = re.compile(r"<parameter=([^>\s]+)>(.*?)</parameter>", re.S)
_FENCE_RE = re.compile(r"```(?:json)?\s*(.*?)```", re.S)


def _schemas(tools: Optional[list[dict]]) -> dict[str, dict]:
    """tool name -> {parameter name -> JSON-schema fragment}."""
    out: dict[str, dict] = {}
    for t in tools or []:
        f = t.get("function", t)
        if isinstance(f, dict) and f.get("name"):
            out[f["name"]] = ((f.get("parameters") or {}).get("properties") or {})
    return out


def _coerce(raw: str, schema: Optional[dict]):
    """A parameter value written as text -> the JSON type its schema asks for (strings stay strings;
    numbers, booleans, arrays and objects are parsed; anything unparsable stays a string)."""
    v = raw.strip("\n")
    typ = (schema or {}).get("type")
    if typ == "string":
        return v
    if typ in ("integer", "number"):
        try:
            f = float(v)
            return int(f) if typ == "integer" and f.is_integer() else f
        except ValueError:
            return v
    if typ == "boolean":
        return {"true": True, "false": False}.get(v.strip().lower(), v)
    if typ in ("array", "object") or typ is None:
        try:
            return json.loads(v)
        except json.JSONDecodeError:
            return v
    return v


def _parse_qwen3_coder(text: str, known, schemas) -> tuple[str, list[ToolCall]]:
    calls: list[ToolCall] = []

    def repl(m: re.Match) -> str:
        name = m.group(1)
        if known is not None and name not in known:
            return m.group(0)
        props = schemas.get(name, {})
        args = {k: _coerce(v, props.get(k)) for k, v in _PARAM_RE.findall(m.group(2))}
        calls.append(ToolCall(function=FunctionCall(name=name, arguments=json.dumps(args))))
        return ""
    rest = _CODER_RE.sub(repl, text)
    return (rest.strip() if calls else text), calls


def _parse_bare_json(text: str, known) -> tuple[str, list[ToolCall]]:
    body = text.strip()
    m = _FENCE_RE.search(body)
    cand = m.group(1).strip() if m else body
    if cand.startswith("<|python_tag|>"):
        cand = cand[len("<|python_tag|>"):].strip()
    try:
        obj = json.loads(cand)
    except json.JSONDecodeError:
        return text, []
    items = obj if isinstance(obj, list) else [obj]
    calls = []
    for it in items:
        if not isinstance(it, dict) or not isinstance(it.get("name"), str) or (known is not None and it["name"] not in known):
            return text, []
        args = it.get("arguments", it.get("parameters", {}))
        calls.append(ToolCall(function=FunctionCall(name=it["name"], arguments=args if isinstance(args, str) else json.dumps(args))))
    rest = (body[: m.start()] + body[m.end():]).strip() if m else ""
    return rest, calls


def parse_tool_calls(text: str, tools: Optional[list[dict]] = None, parser: str = "qwen25") -> tuple[str, list[ToolCall]]:
    """Returns (text without the tool-call blocks, parsed calls). Blocks that are not valid
    or name an unknown tool stay in the text."""
    known = None
    if tools:
        known = {t.get("function", t).get("name") for t in tools}
    if parser in ("qwen3_coder", "qwen3-coder"):
        return _parse_qwen3_coder(text, known, _schemas(tools))
    if parser in ("json", "llama3_json"):
        return _parse_bare_json(text, known)
    if parser == "auto":
        for fn in (lambda: _parse_qwen3_coder(text, known, _schemas(tools)), lambda: parse_tool_calls(text, tools, "qwen25"),
                   lambda: _parse_bare_json(text, known)):
            rest, calls = fn()
            if calls:
                return rest, calls
        return text, []
    if parser not in ("qwen25", "qwen", "hermes", "qwen3"):
        raise ValueError(f"unknown tool-call parser '{parser}'")
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
