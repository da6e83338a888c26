"""Ready-made agent workflows on the OpenAI-compatible surface (in-process client or per-episode proxy session).

Every agent has ``async run(data, **extra) -> reward``: ``extra`` carries ``client`` (the recording in-process client)
and, in proxy mode, ``base_url`` / ``api_key`` of the episode's session, so the same class runs with the SDK of its
ecosystem over HTTP or without any SDK in the trainer's process. Give the class (or ``module.Class`` as a string) as
``workflow`` to the trainer; the adapter in ``rollout/workflows/agent.py`` turns the returned reward and the recorded
calls into training tensors.

Reference: ``areal/workflow/{openai,anthropic,openai_agent,langchain}/*``.
"""
from .math_agents import (AnthropicMathAgent, LangChainMathAgent, MathAgent, MultiTurnMathAgent, OpenAIAgentsMathAgent,  # noqa: F401
                          math_reward)

__all__ = ["MathAgent", "MultiTurnMathAgent", "AnthropicMathAgent", "OpenAIAgentsMathAgent", "LangChainMathAgent", "math_reward"]
