"""In-process client with the shape of the Anthropic SDK (``client.messages.create``) over :class:`ArealOpenAI`.

Agent code written against ``anthropic.AsyncAnthropic`` runs unchanged with this object in its place: requests are
translated to chat completions (system prompt, text / tool_use / tool_result content blocks, tool schemas, stop
sequences), answered by the rollout engine, recorded token by token for training, and translated back into a message
object (``content`` blocks, ``stop_reason``, ``usage``). Rewards and export go through the wrapped client. Reference:
the Anthropic workflow of ``areal/workflow/anthropic/`` and the ``/v1/messages`` route of the proxy.
"""
from __future__ import annotations

from types import SimpleNamespace
from typing import Any, Optional

from .client import ArealOpenAI
from .proxy import anthropic_to_openai, openai_to_anthropic


def _as_object(msg: dict) -> SimpleNamespace:
    """The reply as attribute-style objects (``resp.content[0].text``, ``resp.usage.output_tokens``), as the SDK gives them."""
    blocks = [SimpleNamespace(**b) for b in msg["content"]]
    return SimpleNamespace(id=msg["id"], type="message", role="assistant", model=msg["model"], content=blocks,
                           stop_reason=msg["stop_reason"], stop_sequence=None, usage=SimpleNamespace(**msg["usage"]),
                           model_dump=lambda: msg, to_dict=lambda: msg)


class _Messages:
    def __init__(self, owner: "ArealAnthropic"):
        self._o = owner

    async def create(self, *, messages: list[dict], max_tokens: int, model: str = "default", system: Any = None,
                     temperature: Optional[float] = None, top_p: Optional[float] = None, tools: Optional[list[dict]] = None,
                     stop_sequences: Optional[list[str]] = None, metadata: Optional[dict] = None, stream: bool = False, **ignored):
        if stream:
            raise NotImplementedError("streaming is served by the HTTP proxy (/v1/messages with stream: true)")
        body = {"messages": messages, "max_tokens": max_tokens, "system": system, "temperature": temperature, "top_p": top_p,
                "tools": tools or [], "stop_sequences": stop_sequences}
        kw = {k: v for k, v in anthropic_to_openai(body).items() if v is not None}
        comp = await self._o.openai.chat.completions.create(model=model, metadata=metadata, **kw)
        return _as_object(openai_to_anthropic(comp))


class ArealAnthropic:
    def __init__(self, engine=None, tokenizer=None, openai_client: Optional[ArealOpenAI] = None, **kw):
        self.openai = openai_client or ArealOpenAI(engine, tokenizer, **kw)
        self.messages = _Messages(self)

    # rewards and export are those of the wrapped client (message ids are its interaction ids)
    def set_reward(self, id: str, reward: float) -> None:
        self.openai.set_reward(id, reward)

    def set_last_reward(self, reward: float) -> None:
        self.openai.set_last_reward(reward)

    def export_interactions(self, style: str = "individual", reward_discount: Optional[float] = None):
        return self.openai.export_interactions(style, reward_discount)

    def to_trajectory(self, style: str = "individual", reward_discount: Optional[float] = None):
        return self.openai.to_trajectory(style, reward_discount)
