"""OpenAI-compatible async client over an inference engine that records, per call, the
token ids, logprobs and weight versions needed for RL training.

    client = ArealOpenAI(engine=engine, tokenizer=tokenizer)
    c = await client.chat.completions.create(messages=[...], max_completion_tokens=256)
    client.set_reward(c.id, 1.0)            # or set_last_reward
    client.apply_reward_discount(0.9)
    trajs = client.export_interactions(style="individual")

Reference: ``areal/experimental/openai/client.py`` (``AsyncCompletionsWithReward.create``
:638-970, ``ArealOpenAI`` :1429-1580). The OpenAI SDK is not a dependency: the returned
objects only mirror the attributes agent code reads.
"""
from __future__ import annotations

import json
import uuid
from typing import Any, Optional

from ..api.cli_args import GenerationHyperparameters
from ..api.io_struct import ModelRequest
from .cache import InteractionCache
from .tool_call_parser import parse_tool_calls, split_reasoning
from .types import ChatCompletion, ChatMessage, Choice, InteractionWithTokenLogpReward, Response, Usage


def render_messages_plain(messages: list[dict], add_generation_prompt: bool = True) -> str:
    """Template-free rendering for tokenizers without a chat template."""
    out = []
    for m in messages:
        c = m.get("content")
        if isinstance(c, list):
            c = "".join(p.get("text", "") if isinstance(p, dict) else str(p) for p in c)
        out.append(f"{m.get('role', 'user')}: {c or ''}\n")
    if add_generation_prompt:
        out.append("assistant: ")
    return "".join(out)


def encode_messages(tokenizer, messages: list[dict], tools: Optional[list[dict]] = None, enable_thinking: Optional[bool] = None,
                    add_generation_prompt: bool = True) -> list[int]:
    if hasattr(tokenizer, "apply_chat_template") and getattr(tokenizer, "chat_template", None):
        kw: dict[str, Any] = {}
        if tools:
            kw["tools"] = tools
        if enable_thinking is not None:
            kw["enable_thinking"] = enable_thinking
        ids = tokenizer.apply_chat_template(messages, tokenize=True, add_generation_prompt=add_generation_prompt, **kw)
        if isinstance(ids, dict):
            ids = ids["input_ids"]
        return list(ids)
    return list(tokenizer.encode(render_messages_plain(messages, add_generation_prompt)))


class _Completions:
    def __init__(self, client: "ArealOpenAI"):
        self._c = client

    async def create(self, *, messages: list[dict], model: str = "default", temperature: Optional[float] = None,
                     top_p: Optional[float] = None, max_tokens: Optional[int] = None, max_completion_tokens: Optional[int] = None,
                     stop: Optional[Any] = None, n: int = 1, tools: Optional[list[dict]] = None, tool_choice: Any = None,
                     frequency_penalty: Optional[float] = None, extra_body: Optional[dict] = None, metadata: Optional[dict] = None,
                     stream: bool = False, **ignored) -> ChatCompletion:
        c = self._c
        if n != 1:
            raise NotImplementedError("n != 1: issue several calls (each is recorded separately)")
        if stream:
            raise NotImplementedError("streaming is served by the HTTP proxy, not the in-process client")
        messages = [dict(m) if isinstance(m, dict) else m.to_dict() for m in messages]
        inter = InteractionWithTokenLogpReward(messages=messages, chat_template_type=c.chat_template_type)
        cid = "chatcmpl-" + uuid.uuid4().hex
        # parent lookup happens on insertion; for concat mode the request's tokens must extend
        # the parent's exact token sequence, so only the new messages are tokenised
        c._cache[cid] = inter
        if c.chat_template_type == "concat" and inter.parent is not None and inter.parent.model_response is not None:
            p = inter.parent.to_tensor_dict()["input_ids"][0].tolist()
            rest = messages[len(inter.parent.full_messages):]
            input_ids = p + c._encode_continuation(rest)
        else:
            input_ids = encode_messages(c.tokenizer, messages, tools, (extra_body or {}).get("enable_thinking", c.enable_thinking))
        g: GenerationHyperparameters = c.gconfig.new(n_samples=1)
        if temperature is not None:
            g.temperature = temperature
            g.greedy = temperature == 0
        if top_p is not None:
            g.top_p = top_p
        mt = max_completion_tokens if max_completion_tokens is not None else max_tokens
        if mt is not None:
            g.max_new_tokens = mt
        if frequency_penalty is not None:
            g.frequency_penalty = frequency_penalty
        if stop:
            g.stop = [stop] if isinstance(stop, str) else list(stop)
        if c.max_total_tokens is not None:
            room = c.max_total_tokens - len(input_ids)
            if room <= 0:
                raise ValueError(f"prompt of {len(input_ids)} tokens leaves no room under max_total_tokens={c.max_total_tokens}")
            g.max_new_tokens = min(g.max_new_tokens, room)
        req = ModelRequest(rid=cid, input_ids=input_ids, gconfig=g, tokenizer=c.tokenizer, metadata=metadata or {})
        resp = await c.engine.agenerate(req)
        out_ids = list(resp.output_tokens)
        eos = getattr(c.tokenizer, "eos_token_id", None)
        text = c.tokenizer.decode(out_ids[:-1] if out_ids and out_ids[-1] == eos else out_ids)
        reasoning, visible = split_reasoning(text)
        content, calls = parse_tool_calls(visible, tools, c.tool_call_parser) if tools else (visible, [])
        finish = "tool_calls" if calls else ("length" if resp.stop_reason == "length" else "stop")
        msg = ChatMessage(role="assistant", content=content, tool_calls=calls or None, reasoning_content=reasoning)
        comp = ChatCompletion(id=cid, model=model, choices=[Choice(0, msg, finish)],
                              usage=Usage(resp.input_len, resp.output_len, resp.input_len + resp.output_len))
        inter.interaction_id = cid
        inter.model_response = resp
        # the training-side conversation keeps the raw text so later turns reproduce the tokens
        raw = {"role": "assistant", "content": text if not calls else content}
        if calls:
            raw["tool_calls"] = msg.to_dict()["tool_calls"]
        inter.output_message_list = [raw]
        inter.completion = comp
        return comp


class _Chat:
    def __init__(self, client):
        self.completions = _Completions(client)


class _Responses:
    def __init__(self, client: "ArealOpenAI"):
        self._c = client

    async def create(self, *, input: Any, instructions: Optional[str] = None, model: str = "default",
                     max_output_tokens: Optional[int] = None, temperature: Optional[float] = None, top_p: Optional[float] = None,
                     tools: Optional[list[dict]] = None, **ignored) -> Response:
        msgs: list[dict] = []
        if instructions:
            msgs.append({"role": "system", "content": instructions})
        if isinstance(input, str):
            msgs.append({"role": "user", "content": input})
        else:
            for it in input:
                if it.get("type") == "function_call_output":
                    msgs.append({"role": "tool", "content": it.get("output", ""), "tool_call_id": it.get("call_id")})
                else:
                    msgs.append({"role": it.get("role", "user"), "content": it.get("content", "")})
        comp = await self._c.chat.completions.create(messages=msgs, model=model, max_completion_tokens=max_output_tokens,
                                                     temperature=temperature, top_p=top_p, tools=tools)
        inter = self._c._cache[comp.id]
        inter.api_type = "response"
        m = comp.choices[0].message
        out = [{"type": "message", "role": "assistant", "content": [{"type": "output_text", "text": m.content or ""}]}]
        for t in m.tool_calls or []:
            out.append({"type": "function_call", "call_id": t.id, "name": t.function.name, "arguments": t.function.arguments})
        return Response(id=comp.id, output_text=m.content or "", output=out, model=model, usage=comp.usage)


class ArealOpenAI:
    def __init__(self, engine, tokenizer, gconfig: Optional[GenerationHyperparameters] = None, chat_template_type: str = "hf",
                 enable_thinking: Optional[bool] = None, max_total_tokens: Optional[int] = None, tool_call_parser: str = "auto", **_):
        if chat_template_type not in ("hf", "concat"):
            raise ValueError("chat_template_type must be 'hf' or 'concat'")
        self.engine, self.tokenizer = engine, tokenizer
        self.gconfig = gconfig or GenerationHyperparameters()
        self.chat_template_type = chat_template_type
        self.enable_thinking = enable_thinking
        self.max_total_tokens = max_total_tokens
        self.tool_call_parser = tool_call_parser
        self._cache = InteractionCache()
        self.chat = _Chat(self)
        self.responses = _Responses(self)

    def _encode_continuation(self, messages: list[dict]) -> list[int]:
        """Tokens that the new (non-assistant) messages add after the parent's sequence."""
        text = render_messages_plain(messages, add_generation_prompt=True)
        if not text.startswith("\n"):
            text = "\n" + text
        return list(self.tokenizer.encode(text))

    # ---- reward API
    def get_interaction(self, id: str) -> Optional[InteractionWithTokenLogpReward]:
        return self._cache.get(id)

    get_completions = get_interaction

    def set_reward(self, id: str, reward: float) -> None:
        self._cache.set_reward(id, reward)

    def set_last_reward(self, reward: float) -> None:
        self._cache.set_last_reward(reward)

    def apply_reward_discount(self, turn_discount: float = 1.0):
        return self._cache.apply_reward_discount(turn_discount)

    def export_interactions(self, style: str = "individual", reward_discount: Optional[float] = None):
        return self._cache.export_interactions(style, reward_discount)

    export_completions = export_interactions

    def to_trajectory(self, style: str = "individual", reward_discount: Optional[float] = None):
        """Exported interactions as ONE padded batch (``None`` if nothing was recorded)."""
        from ..utils.data import concat_padded_tensors

        inter = self.export_interactions(style, reward_discount)
        ts = [v.to_tensor_dict() for v in inter.values() if v.has_tensor_data]
        return concat_padded_tensors(ts) if ts else None
