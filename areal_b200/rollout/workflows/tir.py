"""Tool-integrated reasoning: the model writes a fenced ``python`` block, generation stops at
the closing fence, the block runs in the sandbox and its output is appended as an
``output`` block that is masked out of the loss; the model then continues. The episode ends
with an answer (no new code block), after ``max_tool_calls`` executions, or at the token budget.

Reference: ``examples/tir/`` (tool-calling loop around ``engine.agenerate`` with stop strings,
tool text excluded from the loss, final answer scored by the math verifier).
"""
from __future__ import annotations

import asyncio
import uuid
from typing import Any, Callable, Optional

import torch

from ...api.cli_args import GenerationHyperparameters
from ...api.io_struct import ModelRequest
from ...api.workflow_api import RolloutWorkflow
from ...infra.sandbox.local import LocalSandbox, SandboxConfig, extract_code_blocks
from ...utils import stats_tracker
from .. import workflow_context as wctx
from .rlvr import default_get_input_ids

FENCE = "```"


class TIRWorkflow(RolloutWorkflow):
    def __init__(self, reward_fn: Callable[..., float], gconfig: GenerationHyperparameters, tokenizer, max_tool_calls: int = 4,
                 sandbox: Optional[LocalSandbox] = None, max_tool_output_chars: int = 1024, get_input_ids_fn: Callable = default_get_input_ids,
                 enable_thinking: bool = False):
        self.reward_fn, self.gconfig, self.tokenizer = reward_fn, gconfig, tokenizer
        self.max_tool_calls = max_tool_calls
        self.sandbox = sandbox or LocalSandbox(SandboxConfig(timeout_s=5.0))
        self.max_tool_output_chars = max_tool_output_chars
        self.get_input_ids_fn, self.enable_thinking = get_input_ids_fn, enable_thinking

    @staticmethod
    def pending_code(text: str) -> Optional[str]:
        """The code of a just-closed ``python`` block at the end of ``text`` (None when the text
        does not end in a closed block)."""
        t = text.rstrip()
        if not t.endswith(FENCE) or t.count(FENCE) % 2:
            return None
        blocks = extract_code_blocks(t + "\n")
        return blocks[-1] if blocks else None

    def _tool_text(self, code: str) -> str:
        r = self.sandbox.run(code)
        out = r.stdout if r.ok else (f"[timed out after {r.seconds:.1f}s]" if r.timed_out else f"[exit code {r.returncode}]\n{r.stdout}{r.stderr[-500:]}")
        out = out[: self.max_tool_output_chars]
        return f"\n{FENCE}output\n{out.rstrip()}\n{FENCE}\n"

    async def arun_episode(self, engine, data: dict[str, Any]) -> Optional[dict[str, torch.Tensor]]:
        tok = self.tokenizer
        seq = list(self.get_input_ids_fn(data, tok, self.enable_thinking))
        n_prompt = len(seq)
        logprobs, loss_mask, versions = [0.0] * n_prompt, [0] * n_prompt, [-1] * n_prompt
        calls, completion = 0, ""
        loop = asyncio.get_running_loop()
        while True:
            room = self.gconfig.max_tokens - len(seq)
            if room <= 0:
                break
            # stop at a closing fence: the block that just ended may be code to run
            g = self.gconfig.new(n_samples=1, max_new_tokens=min(self.gconfig.max_new_tokens, room), stop=[FENCE + "\n"])
            resp = await engine.agenerate(ModelRequest(rid=uuid.uuid4().hex, input_ids=list(seq), gconfig=g, tokenizer=tok))
            seq += resp.output_tokens
            logprobs += resp.output_logprobs
            loss_mask += [1] * resp.output_len
            versions += resp.output_versions
            text = tok.decode(resp.output_tokens)
            completion += text
            code = self.pending_code(completion)
            if code is None or calls >= self.max_tool_calls or resp.stop_reason == "length":
                break
            calls += 1
            tool = await loop.run_in_executor(None, self._tool_text, code)
            ids = list(tok.encode(tool))
            if len(seq) + len(ids) >= self.gconfig.max_tokens:
                break
            seq += ids
            logprobs += [0.0] * len(ids)
            loss_mask += [0] * len(ids)
            versions += [-1] * len(ids)
            completion += tool
        kw = {k: v for k, v in data.items() if k not in ("input_ids", "messages", "prompt")}
        r = self.reward_fn(tok.decode(seq[:n_prompt]), completion, seq[:n_prompt], seq[n_prompt:], **kw)
        if asyncio.iscoroutine(r):
            r = await r
        stats_tracker.get(wctx.stat_scope()).scalar(reward=float(r), tool_calls=float(calls))
        L = len(seq)
        return {
            "input_ids": torch.tensor(seq, dtype=torch.long).unsqueeze(0),
            "loss_mask": torch.tensor(loss_mask, dtype=torch.int32).unsqueeze(0),
            "logprobs": torch.tensor(logprobs, dtype=torch.float32).unsqueeze(0),
            "versions": torch.tensor(versions, dtype=torch.int32).unsqueeze(0),
            "attention_mask": torch.ones(1, L, dtype=torch.bool),
            "rewards": torch.tensor([float(r)], dtype=torch.float32),
        }
