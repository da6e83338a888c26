"""Single-turn RL-with-verifiable-reward workflow: generate ``n_samples`` completions of one
prompt, score each with a reward function, return the group as one padded batch.

Trajectory layout (reference ``areal/workflow/rlvr.py:164-180``): ``input_ids`` (prompt +
completion), ``loss_mask`` (0 prompt / 1 generated), ``logprobs`` (0 on the prompt, behaviour
log-prob per generated token), ``versions`` (-1 on the prompt, generating weight version per
token), ``turn_ids`` (-1 prompt, 0 for the single turn), ``attention_mask``, ``rewards``.
"""
from __future__ import annotations

import asyncio
import uuid
from typing import Any, Callable, Optional

import torch

from ...api.cli_args import GenerationHyperparameters
from ...api.io_struct import ModelRequest
from ...api.reward_api import AsyncRewardWrapper
from ...api.workflow_api import RolloutWorkflow
from ...utils import data as D
from ...utils import logging as alog
from ...utils import stats_tracker
from .. import workflow_context as wctx


def default_get_input_ids(data: dict[str, Any], tokenizer, enable_thinking: bool = False) -> list[int]:
    if "input_ids" in data:
        ids = data["input_ids"]
        return ids.tolist() if torch.is_tensor(ids) else list(ids)
    if tokenizer is None:
        raise ValueError("data has no 'input_ids' and no tokenizer was given")
    if "messages" in data:
        return list(tokenizer.apply_chat_template(data["messages"], tokenize=True, add_generation_prompt=True,
                                                  enable_thinking=enable_thinking))
    return list(tokenizer.encode(data["prompt"]))


logger = alog.getLogger("workflow")


class RLVRWorkflow(RolloutWorkflow):
    def __init__(self, reward_fn: Callable[..., float], gconfig: GenerationHyperparameters, tokenizer=None,
                 enable_thinking: bool = False, get_input_ids_fn: Callable = default_get_input_ids,
                 reward_in_process: bool = False, reward_timeout: float = 15.0):
        if isinstance(reward_fn, str):  # import path: how a workflow is described to a remote worker
            from ...utils.dynamic_import import import_from_string

            reward_fn = import_from_string(reward_fn)
        if isinstance(get_input_ids_fn, str):
            from ...utils.dynamic_import import import_from_string

            get_input_ids_fn = import_from_string(get_input_ids_fn)
        self.gconfig = gconfig
        self.tokenizer = tokenizer
        self.enable_thinking = enable_thinking
        self.get_input_ids_fn = get_input_ids_fn
        self.reward_fn = reward_fn
        self._reward_in_process = reward_in_process
        self._areward = None if reward_in_process else AsyncRewardWrapper(reward_fn, timeout_seconds=reward_timeout)

    async def _reward(self, prompt_str, completion_str, prompt_ids, completion_ids, data):
        kw = {k: v for k, v in data.items() if k not in ("input_ids", "messages", "prompt", "max_new_tokens_per_sample")}
        if self._reward_in_process:
            r = self.reward_fn(prompt_str, completion_str, prompt_ids, completion_ids, **kw)
            if asyncio.iscoroutine(r):
                r = await r
            return float(r)
        return await self._areward(prompt_str, completion_str, prompt_ids, completion_ids, **kw)

    async def _one_sample(self, engine, input_ids: list[int], data, gconfig) -> dict[str, torch.Tensor]:
        req = ModelRequest(rid=uuid.uuid4().hex, input_ids=input_ids, gconfig=gconfig, tokenizer=self.tokenizer)
        resp = await engine.agenerate(req)
        prompt_str = completion_str = None
        if self.tokenizer is not None:
            prompt_str = self.tokenizer.decode(input_ids)
            completion_str = self.tokenizer.decode(resp.output_tokens)
        reward = await self._reward(prompt_str, completion_str, resp.input_tokens, resp.output_tokens, data)
        stats_tracker.get(wctx.stat_scope()).scalar(reward=reward, gen_len=len(resp.output_tokens))
        seq = resp.input_tokens + resp.output_tokens
        n_in, n_out = resp.input_len, resp.output_len
        return dict(
            input_ids=torch.tensor(seq, dtype=torch.int32).unsqueeze(0),
            loss_mask=torch.tensor([0] * n_in + [1] * n_out, dtype=torch.int32).unsqueeze(0),
            logprobs=torch.tensor([0.0] * n_in + resp.output_logprobs, dtype=torch.float32).unsqueeze(0),
            versions=torch.tensor([-1] * n_in + resp.output_versions, dtype=torch.int32).unsqueeze(0),
            turn_ids=torch.tensor([-1] * n_in + [0] * n_out, dtype=torch.int32).unsqueeze(0),
            attention_mask=torch.ones(1, len(seq), dtype=torch.bool),
            rewards=torch.tensor([float(reward)], dtype=torch.float32),
        )

    async def arun_episode(self, engine, data: dict[str, Any]) -> Optional[dict[str, Any]]:
        input_ids = self.get_input_ids_fn(data, self.tokenizer, self.enable_thinking)
        n = max(1, self.gconfig.n_samples)
        g1 = self.gconfig.new(n_samples=1)
        if "max_new_tokens" in data:  # per-prompt response budget (forced-length experiments)
            g1 = g1.new(max_new_tokens=int(data["max_new_tokens"]))
        per = data.get("max_new_tokens_per_sample")     # forced-length experiments: one budget per sample of the group
        gs = [g1.new(max_new_tokens=int(per[i % len(per)])) if per else g1 for i in range(n)]
        samples = await asyncio.gather(*[self._one_sample(engine, input_ids, data, gs[i]) for i in range(n)])
        return D.concat_padded_tensors(list(samples))


class GroupedRolloutWorkflow(RolloutWorkflow):
    """Runs ``group_size`` episodes of an inner workflow concurrently (each with its own ``sample_idx`` in the workflow
    context) and concatenates them.

    * ``drop_incomplete_group``: a group in which any episode failed (returned ``None``) is dropped as a whole, so
      group-level baselines always see ``group_size`` samples; the trainer's batch preparation then takes another prompt.
      Otherwise the remaining episodes are kept (variable group size).
    * ``reward_normalization``: every episode's reward (its last one, when an episode exports several sequences) is
      replaced by its z-score inside the group; the raw values stay in ``original_rewards``. A group with a missing reward
      is dropped, so the normalisation base is always the configured size.

    Reference: ``areal/infra/remote_inf_engine.py:70-206``; the two switches are ``gconfig.drop_incomplete_group`` and
    ``gconfig.reward_normalization`` (see :meth:`from_gconfig`)."""

    def __init__(self, workflow: RolloutWorkflow, group_size: int, reward_normalization: bool = False, drop_incomplete_group: bool = False,
                 serialize_group_samples: bool = False):
        """``serialize_group_samples``: the episodes of a group run one after another instead of concurrently (an agent
        whose tools hold per-prompt state, or a server whose prefix cache should see the first sample finish before
        the others start; ``rollout.serialize_group_samples``)."""
        if group_size < 1:
            raise ValueError(f"group_size must be >= 1, got {group_size}")
        self.workflow, self.group_size = workflow, group_size
        self.reward_normalization, self.drop_incomplete_group = reward_normalization, drop_incomplete_group
        self.serialize_group_samples = serialize_group_samples

    @classmethod
    def from_gconfig(cls, workflow: RolloutWorkflow, gconfig: GenerationHyperparameters, rollout_config=None) -> "GroupedRolloutWorkflow":
        return cls(workflow, max(1, gconfig.n_samples), bool(getattr(gconfig, "reward_normalization", False)),
                   bool(getattr(gconfig, "drop_incomplete_group", False)), bool(getattr(rollout_config, "serialize_group_samples", False)))

    async def arun_episode(self, engine, data):
        parent = wctx.get()

        async def one(i: int):
            with wctx.scoped(is_eval=parent.is_eval, task_id=parent.task_id, sample_idx=i):
                return await self.workflow.arun_episode(engine, data)

        if self.serialize_group_samples:
            res = [await one(i) for i in range(self.group_size)]
        else:
            res = await asyncio.gather(*[one(i) for i in range(self.group_size)])
        ok = [r for r in res if r is not None]
        if not ok:
            return None
        if len(ok) < len(res) and (self.drop_incomplete_group or self.reward_normalization):
            logger.warning("grouped rollout: %d of %d episodes failed, dropping the group", len(res) - len(ok), len(res))
            return None
        if self.reward_normalization and self.group_size > 1:
            last = torch.stack([r["rewards"].float().reshape(-1)[-1] for r in ok])
            z = (last - last.mean()) / (last.std(unbiased=False) + 1e-8)
            for r, v in zip(ok, z):
                r["original_rewards"] = r["rewards"].clone()
                r["rewards"] = torch.full_like(r["rewards"].float(), float(v))
        return D.concat_padded_tensors(ok)
