"""Online training: episodes come from outside users instead of a dataset.

An outside program opens a session on the trainer's OpenAI-compatible proxy (``POST /rl/start_session`` with the admin
key), talks to the model with the session key as its API key (any OpenAI / Anthropic SDK, an agent framework, a chat
loop), scores what happened (``POST /rl/set_reward``) and closes the session (``POST /rl/end_session``). Each call of
:meth:`OnlineSessionWorkflow.arun_episode` waits for ONE such finished session and returns its recorded turns as a
trajectory; the data item it is given is ignored (the data loader of an online run yields placeholders). Staleness
control, batching and the PPO update are those of any other workflow.

Reference: ``areal/experimental/openai/proxy/online_agent.py`` and the ``mode="online"`` path of its proxy workflow;
``examples/hermes`` / ``examples/openclaw`` drive it from outside.
"""
from __future__ import annotations

import asyncio
from typing import Any, Optional

from ...api.workflow_api import RolloutWorkflow
from ...utils import stats_tracker
from .. import workflow_context as wctx


class OnlineSessionWorkflow(RolloutWorkflow):
    def __init__(self, proxy, export_style: str = "individual", turn_discount: float = 1.0, timeout: float = 3600.0,
                 default_reward: Optional[float] = None):
        """``proxy``: the running :class:`~areal_b200.openai.proxy.OpenAIProxyServer` outside users talk to.
        ``default_reward``: reward of a session that ended without one (``None``: such a session is dropped)."""
        self.proxy, self.export_style, self.turn_discount = proxy, export_style, turn_discount
        self.timeout, self.default_reward = timeout, default_reward

    async def arun_episode(self, engine, data: dict[str, Any]):
        loop = asyncio.get_running_loop()
        key = await loop.run_in_executor(None, self.proxy.wait_for_completed_session, self.timeout)
        if key is None:
            return None                                  # nobody finished a session in time: the episode is rejected
        sess = self.proxy.pop_session(key)
        if sess is None or len(sess.client._cache) == 0:
            return None
        client = sess.client
        if not any(it.reward is not None for it in client._cache.values()):
            if self.default_reward is None:
                return None
            client.set_last_reward(float(self.default_reward))
        client.apply_reward_discount(self.turn_discount)
        traj = client.to_trajectory(self.export_style)
        if traj is not None:
            stats_tracker.get(wctx.stat_scope()).scalar(reward=float(traj["rewards"].float().mean()), n_turns=float(len(client._cache)))
        return traj
