"""Multi-turn self-correction workflow: the model answers, a reward function judges; on a
wrong answer a fixed feedback message is appended (not trained on) and the model tries again,
up to ``max_turns``. The final reward is discounted by ``turn_discount`` per retry.
Reference: ``areal/workflow/multi_turn.py``."""
from __future__ import annotations

import uuid
from typing import Any, Callable, Optional

import torch

from ...api.cli_args import GenerationHyperparameters
from ...api.io_struct import ModelRequest
from ...api.reward_api import AsyncRewardWrapper
from ...api.workflow_api import RolloutWorkflow
from ...utils import stats_tracker
from .. import workflow_context as wctx

DEFAULT_FEEDBACK = "Your answer is either wrong or not parsable to the reward function. Please try to answer it again."


class MultiTurnWorkflow(RolloutWorkflow):
    def __init__(self, reward_fn: Callable[..., float], gconfig: GenerationHyperparameters, tokenizer, max_turns: int = 3,
                 turn_discount: float = 0.9, feedback: str = DEFAULT_FEEDBACK, reward_in_process: bool = False,
                 success_threshold: float = 0.0):
        if isinstance(reward_fn, str):
            from ...utils.dynamic_import import import_from_string

            reward_fn = import_from_string(reward_fn)
        self.reward_fn = reward_fn
        self.gconfig = gconfig.new(n_samples=1)
        self.tokenizer = tokenizer
        self.max_turns = max_turns
        self.turn_discount = turn_discount
        self.feedback = feedback
        self.success_threshold = success_threshold
        self._in_process = reward_in_process
        self._areward = None if reward_in_process else AsyncRewardWrapper(reward_fn)

    def _encode_prompt(self, data) -> list[int]:
        if "input_ids" in data:
            return list(data["input_ids"])
        from ...openai.client import encode_messages

        return encode_messages(self.tokenizer, data["messages"])

    def _encode_feedback(self) -> list[int]:
        from ...openai.client import render_messages_plain

        return list(self.tokenizer.encode("\n" + render_messages_plain([{"role": "user", "content": self.feedback}])))

    async def arun_episode(self, engine, data: dict[str, Any]) -> Optional[dict[str, torch.Tensor]]:
        seq = self._encode_prompt(data)
        n_prompt = len(seq)
        logprobs, loss_mask, versions = [0.0] * n_prompt, [0] * n_prompt, [-1] * n_prompt
        discount, reward, turns = 1.0, 0.0, 0
        kw = {k: v for k, v in data.items() if k not in ("input_ids", "messages", "prompt")}
        fb = self._encode_feedback()
        for turn in range(self.max_turns):
            room = self.gconfig.max_tokens - len(seq)
            if room <= 0:
                break
            g = self.gconfig.new(max_new_tokens=min(self.gconfig.max_new_tokens, room))
            resp = await engine.agenerate(ModelRequest(rid=uuid.uuid4().hex, input_ids=list(seq), gconfig=g, tokenizer=self.tokenizer))
            turns += 1
            seq += resp.output_tokens
            logprobs += resp.output_logprobs
            loss_mask += [1] * resp.output_len
            versions += resp.output_versions
            prompt_str = self.tokenizer.decode(seq[:n_prompt])
            completion_str = self.tokenizer.decode(resp.output_tokens)
            if self._in_process:
                reward = float(self.reward_fn(prompt_str, completion_str, seq[:n_prompt], resp.output_tokens, **kw))
            else:
                reward = float(await self._areward(prompt_str, completion_str, seq[:n_prompt], resp.output_tokens, **kw))
            if reward > self.success_threshold or turn == self.max_turns - 1:
                break
            if len(seq) + len(fb) >= self.gconfig.max_tokens:
                break
            seq += fb
            logprobs += [0.0] * len(fb)
            loss_mask += [0] * len(fb)
            versions += [-1] * len(fb)
            discount *= self.turn_discount
        final = reward * discount
        stats_tracker.get(wctx.stat_scope()).scalar(reward=final, num_turns=float(turns))
        L = len(seq)
        return {
            "input_ids": torch.tensor(seq, dtype=torch.long).unsqueeze(0),
            "loss_mask": torch.tensor(loss_mask, dtype=torch.int32).unsqueeze(0),
            "logprobs": torch.tensor(logprobs, dtype=torch.float32).unsqueeze(0),
            "versions": torch.tensor(versions, dtype=torch.int32).unsqueeze(0),
            "attention_mask": torch.ones(1, L, dtype=torch.bool),
            "rewards": torch.tensor([final], dtype=torch.float32),
        }
