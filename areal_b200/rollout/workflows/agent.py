"""Adapter that runs agent-style user code as a rollout workflow.

The agent receives an OpenAI-compatible client (``extra_kwargs['client']``; for agents that
only speak HTTP also ``base_url`` / ``api_key`` of a per-episode proxy session) and returns a
reward: a float (assigned to the last model call), a dict ``{completion_id: reward}``, or
``None`` (episode rejected). Token capture, reward discounting and export to training
tensors happen here. Reference: ``areal/infra/workflow_executor.py`` agent path and
``areal/experimental/openai/proxy/*``.
"""
from __future__ import annotations

import inspect
from typing import Any, Optional

from ...api.workflow_api import RolloutWorkflow
from ...openai.client import ArealOpenAI
from ...utils import stats_tracker
from .. import workflow_context as wctx


class AgentRolloutAdapter(RolloutWorkflow):
    def __init__(self, agent, config=None, tokenizer=None, gconfig=None, export_style: str = "individual",
                 turn_discount: float = 1.0, chat_template_type: Optional[str] = None, proxy=None):
        self.agent = agent
        self.config = config
        self.tokenizer = tokenizer if tokenizer is not None else getattr(agent, "tokenizer", None)
        self.gconfig = gconfig if gconfig is not None else getattr(agent, "gconfig", None)
        self.export_style = getattr(agent, "export_style", export_style)
        self.turn_discount = getattr(agent, "turn_discount", turn_discount)
        self.chat_template_type = chat_template_type or ("concat" if self.export_style == "concat" else "hf")
        self.proxy = proxy

    async def arun_episode(self, engine, data: dict[str, Any]):
        if self.tokenizer is None:
            raise ValueError("agent workflows need a tokenizer (give one to the adapter or set agent.tokenizer)")
        client = ArealOpenAI(engine, self.tokenizer, gconfig=self.gconfig, chat_template_type=self.chat_template_type)
        extra: dict[str, Any] = {"client": client}
        session = None
        if self.proxy is not None:
            session = self.proxy.start_session(client)
            extra.update(base_url=self.proxy.base_url, api_key=session)
            try:
                extra["http_client"] = wctx.get_httpx_client()      # one connection pool per event loop, not per episode
            except ImportError:
                pass
        try:
            params = inspect.signature(self.agent.run).parameters
            if not any(p.kind == inspect.Parameter.VAR_KEYWORD for p in params.values()):
                extra = {k: v for k, v in extra.items() if k in params}
            r = self.agent.run(data, **extra)
            if inspect.isawaitable(r):
                r = await r
        finally:
            if session is not None:
                self.proxy.end_session(session)
        if r is None or len(client._cache) == 0:
            return None
        if isinstance(r, dict):
            for cid, rew in r.items():
                client.set_reward(cid, float(rew))
        else:
            client.set_last_reward(float(r))
        client.apply_reward_discount(self.turn_discount)
        traj = client.to_trajectory(self.export_style)
        if traj is not None:
            stats_tracker.get(wctx.stat_scope()).scalar(reward=float(traj["rewards"].float().mean()),
                                                        n_turns=float(len(client._cache)))
        return traj
