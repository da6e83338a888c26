"""Math agents: one-shot, retry-with-feedback, Anthropic Messages, OpenAI Agents SDK, LangChain.

The reward is the symbolic comparison of the final answer with the record's ``answer``
(``areal_b200/reward/math_verify.py``). Reference: ``areal/workflow/openai/math_agent.py`` (MathAgent,
MultiTurnMathAgent), ``areal/workflow/anthropic/math_agent.py``, ``areal/workflow/openai_agent/math_agent.py``,
``areal/workflow/langchain/math_agent.py``.
"""
from __future__ import annotations

import os
from typing import Any, Optional

from ..api.workflow_api import AgentWorkflow


def math_reward(completion: Optional[str], answer: Any) -> float:
    from ..reward import get_math_verify_worker

    if not completion:
        return 0.0
    return float(get_math_verify_worker().verify(str(completion), str(answer)))


def _messages_of(data: dict) -> list[dict]:
    m = data.get("messages_chat") or data.get("messages") or data.get("question") or data.get("prompt")
    return [{"role": "user", "content": m}] if isinstance(m, str) else [dict(x) for x in m]


def _sampling_kwargs(kw: dict) -> dict:
    """``max_new_tokens`` of the training configs is ``max_tokens`` on the wire; agent-only keys are dropped."""
    kw = dict(kw)
    n = kw.pop("max_new_tokens", None)
    kw.pop("max_turns", None)
    if n is not None and "max_tokens" not in kw:
        kw["max_tokens"] = n
    return kw


class _ChatCaller:
    """``chat(messages, **kw) -> text`` through whichever handle the episode was given: the in-process client, or the
    ``openai`` SDK pointed at the session's proxy URL."""

    def __init__(self, extra: dict):
        self.client = extra.get("client")
        self.base_url = extra.get("base_url") or os.getenv("OPENAI_BASE_URL")
        self.api_key = extra.get("api_key") or os.getenv("OPENAI_API_KEY")
        self.http_client = extra.get("http_client")
        self._sdk = None

    async def chat(self, messages: list[dict], **kw) -> str:
        if self.base_url and extra_wants_http(self):
            if self._sdk is None:
                from openai import AsyncOpenAI

                self._sdk = AsyncOpenAI(base_url=self.base_url, api_key=self.api_key, http_client=self.http_client, max_retries=0)
            comp = await self._sdk.chat.completions.create(messages=messages, model="default", **kw)
            return comp.choices[0].message.content or ""
        comp = await self.client.chat.completions.create(messages=messages, **kw)
        return comp.choices[0].message.content or ""


def extra_wants_http(c: "_ChatCaller") -> bool:
    """Over HTTP when there is a session URL and either no in-process client or ``AREAL_AGENT_HTTP=1``."""
    return c.client is None or os.getenv("AREAL_AGENT_HTTP", "0") == "1"


class MathAgent(AgentWorkflow):
    """One model call, one reward."""

    def __init__(self, **kwargs):
        self.kwargs = _sampling_kwargs(kwargs)

    async def run(self, data: dict[str, Any], **extra) -> float:
        text = await _ChatCaller(extra).chat(_messages_of(data), **self.kwargs)
        return math_reward(text, data["answer"])


class MultiTurnMathAgent(AgentWorkflow):
    """Up to ``max_turns`` attempts: after a wrong answer the conversation goes on with a short feedback message. The
    reward of the episode is that of the last attempt (earlier turns are discounted by the adapter's ``turn_discount``)."""

    feedback = "Your answer is either wrong or not parsable to the reward function. You may misunderstand the original question. " \
               "Please carefully read the original question, check the previous errors, and try to answer it again."

    def __init__(self, max_turns: int = 8, **kwargs):
        self.max_turns = int(max_turns)
        self.kwargs = _sampling_kwargs(kwargs)

    async def run(self, data: dict[str, Any], **extra) -> float:
        caller, messages, reward = _ChatCaller(extra), _messages_of(data), 0.0
        for _ in range(self.max_turns):
            text = await caller.chat(messages, **self.kwargs)
            reward = math_reward(text, data["answer"])
            if reward >= 1.0:
                break
            messages += [{"role": "assistant", "content": text}, {"role": "user", "content": self.feedback}]
        return reward


class AnthropicMathAgent(AgentWorkflow):
    """The same task through the Anthropic Messages shape: the ``anthropic`` SDK against the session's proxy URL
    (``/v1/messages``), or the in-process Anthropic-shaped client over the recording client."""

    def __init__(self, max_tokens: int = 1024, system: Optional[str] = None, **kwargs):
        self.max_tokens, self.system = int(kwargs.pop("max_new_tokens", max_tokens)), system
        self.kwargs = {k: v for k, v in kwargs.items() if k not in ("max_turns",)}

    async def run(self, data: dict[str, Any], **extra) -> float:
        messages = [m for m in _messages_of(data) if m["role"] != "system"]
        kw = dict(self.kwargs, max_tokens=self.max_tokens, messages=messages)
        if self.system:
            kw["system"] = self.system
        client, base_url = extra.get("client"), extra.get("base_url")
        if base_url and (client is None or os.getenv("AREAL_AGENT_HTTP", "0") == "1"):
            from anthropic import AsyncAnthropic

            root = base_url[:-3] if base_url.rstrip("/").endswith("/v1") else base_url      # the SDK appends /v1/messages itself
            sdk = AsyncAnthropic(base_url=root.rstrip("/"), api_key=extra.get("api_key"), max_retries=0, http_client=extra.get("http_client"))
            msg = await sdk.messages.create(model="default", **kw)
            text = "".join(b.text for b in msg.content if getattr(b, "type", "") == "text")
        else:
            from ..openai.anthropic_client import ArealAnthropic

            msg = await ArealAnthropic(openai_client=client).messages.create(**kw)
            text = "".join(b.text for b in msg.content if b.type == "text")
        return math_reward(text, data["answer"])


class OpenAIAgentsMathAgent(AgentWorkflow):
    """An agent of the OpenAI Agents SDK (``agents``) with arithmetic tools, run against the session's proxy URL; the
    SDK drives the tool-call loop, every model call it makes is recorded by the proxy."""

    instructions = "Solve the problem step by step. Use the tools for arithmetic. Put the final answer in \\boxed{}."

    def __init__(self, max_turns: int = 8, **kwargs):
        self.max_turns = int(max_turns)
        self.kwargs = _sampling_kwargs(kwargs)

    async def run(self, data: dict[str, Any], **extra) -> float:
        from agents import Agent, ModelSettings, OpenAIProvider, RunConfig, Runner, function_tool
        from openai import AsyncOpenAI

        base_url = extra.get("base_url") or os.getenv("OPENAI_BASE_URL")
        if not base_url:
            raise ValueError("the Agents-SDK agent talks HTTP: run it in proxy mode (a session base_url is required)")

        @function_tool
        def add(a: float, b: float) -> float:
            """Sum of two numbers."""
            return a + b

        @function_tool
        def multiply(a: float, b: float) -> float:
            """Product of two numbers."""
            return a * b

        sdk = AsyncOpenAI(base_url=base_url, api_key=extra.get("api_key") or os.getenv("OPENAI_API_KEY"), http_client=extra.get("http_client"),
                          max_retries=0)
        settings = ModelSettings(**{k: v for k, v in self.kwargs.items() if k in ("temperature", "top_p", "max_tokens")})
        agent = Agent(name="math", instructions=self.instructions, tools=[add, multiply], model_settings=settings)
        cfg = RunConfig(model_provider=OpenAIProvider(openai_client=sdk, use_responses=False), tracing_disabled=True)
        msgs = _messages_of(data)
        res = await Runner.run(agent, input=msgs[-1]["content"], run_config=cfg, max_turns=self.max_turns)
        return math_reward(str(res.final_output), data["answer"])


class LangChainMathAgent(AgentWorkflow):
    """``langchain_openai.ChatOpenAI`` pointed at the session's proxy URL (needs the ``langchain-openai`` package)."""

    def __init__(self, **kwargs):
        self.kwargs = _sampling_kwargs(kwargs)

    async def run(self, data: dict[str, Any], **extra) -> float:
        try:
            from langchain_openai import ChatOpenAI
        except ImportError as e:
            raise ImportError("LangChainMathAgent needs the langchain-openai package") from e
        base_url = extra.get("base_url") or os.getenv("OPENAI_BASE_URL")
        llm = ChatOpenAI(model="default", base_url=base_url, api_key=extra.get("api_key") or os.getenv("OPENAI_API_KEY"), max_retries=0,
                         **{k: v for k, v in self.kwargs.items() if k in ("temperature", "top_p", "max_tokens")})
        out = await llm.ainvoke([(m["role"], m["content"]) for m in _messages_of(data)])
        return math_reward(getattr(out, "content", str(out)), data["answer"])
