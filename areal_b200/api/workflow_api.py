"""Rollout workflow contract (reference: ``areal/api/workflow_api.py:14-115``).

A workflow turns one dataset item into one training trajectory (or several) by talking to
an :class:`InferenceEngine`. ``arun_episode`` returns a dict of ``[1, L]`` tensors (see
``areal_b200.rollout.workflows.rlvr``), ``None`` to reject the sample, or a dict of
interaction records when driven through the OpenAI-compatible client.
"""
from __future__ import annotations

import abc
import asyncio
from typing import TYPE_CHECKING, Any, Optional, Union

if TYPE_CHECKING:  # pragma: no cover
    from .engine_api import InferenceEngine


class RolloutWorkflow(abc.ABC):
    @abc.abstractmethod
    async def arun_episode(self, engine: "InferenceEngine", data: dict[str, Any]) -> Optional[dict[str, Any]]:
        raise NotImplementedError


class AgentWorkflow(abc.ABC):
    """Deprecated agent-style interface: ``run`` receives an OpenAI-compatible base URL /
    client and returns a reward (or per-completion rewards); token capture happens in the
    proxy."""

    @abc.abstractmethod
    async def run(self, data: dict[str, Any], **extra_kwargs) -> Union[float, dict[str, float], None]:
        raise NotImplementedError


WorkflowLike = Union[RolloutWorkflow, type, str, AgentWorkflow]


def run_sync(coro):
    """Runs a coroutine to completion from synchronous code (new loop if needed)."""
    try:
        asyncio.get_running_loop()
    except RuntimeError:
        return asyncio.run(coro)
    import concurrent.futures

    with concurrent.futures.ThreadPoolExecutor(max_workers=1) as ex:
        return ex.submit(asyncio.run, coro).result()
