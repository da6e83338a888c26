"""Records of the OpenAI-compatible client: completion objects handed to agent code and the
token-level bookkeeping kept for training. Reference: ``areal/experimental/openai/types.py``
(``InteractionWithTokenLogpReward`` :36, ``to_tensor_dict`` :144)."""
from __future__ import annotations

import time
import uuid
from dataclasses import dataclass, field
from typing import Any, Optional

import torch

from ..api.io_struct import ModelResponse


# ---- what agent code sees (shape of the OpenAI python SDK's objects) -----------------------
@dataclass
class FunctionCall:
    name: str = ""
    arguments: str = "{}"


@dataclass
class ToolCall:
    id: str = field(default_factory=lambda: "call_" + uuid.uuid4().hex[:24])
    type: str = "function"
    function: FunctionCall = field(default_factory=FunctionCall)


@dataclass
class ChatMessage:
    role: str = "assistant"
    content: Optional[str] = None
    tool_calls: Optional[list[ToolCall]] = None
    reasoning_content: Optional[str] = None

    def to_dict(self) -> dict:
        d: dict[str, Any] = {"role": self.role, "content": self.content}
        if self.tool_calls:
            d["tool_calls"] = [{"id": t.id, "type": t.type, "function": {"name": t.function.name, "arguments": t.function.arguments}}
                               for t in self.tool_calls]
        return d

    model_dump = to_dict


@dataclass
class Choice:
    index: int = 0
    message: ChatMessage = field(default_factory=ChatMessage)
    finish_reason: str = "stop"
    logprobs: Any = None


@dataclass
class Usage:
    prompt_tokens: int = 0
    completion_tokens: int = 0
    total_tokens: int = 0


@dataclass
class ChatCompletion:
    id: str = field(default_factory=lambda: "chatcmpl-" + uuid.uuid4().hex)
    choices: list[Choice] = field(default_factory=list)
    created: int = field(default_factory=lambda: int(time.time()))
    model: str = "default"
    object: str = "chat.completion"
    usage: Usage = field(default_factory=Usage)

    def to_dict(self) -> dict:
        return {"id": self.id, "object": self.object, "created": self.created, "model": self.model,
                "choices": [{"index": c.index, "finish_reason": c.finish_reason, "message": c.message.to_dict()} for c in self.choices],
                "usage": {"prompt_tokens": self.usage.prompt_tokens, "completion_tokens": self.usage.completion_tokens,
                          "total_tokens": self.usage.total_tokens}}

    model_dump = to_dict


@dataclass
class Response:
    """Object of the ``responses`` API."""
    id: str = field(default_factory=lambda: "resp-" + uuid.uuid4().hex)
    output_text: str = ""
    output: list[dict] = field(default_factory=list)
    created_at: float = field(default_factory=time.time)
    model: str = "default"
    usage: Usage = field(default_factory=Usage)


# ---- what training sees --------------------------------------------------------------------
@dataclass
class InteractionWithTokenLogpReward:
    """One model call with everything needed to train on it."""

    interaction_id: Optional[str] = None
    messages: list[dict] = field(default_factory=list)            # the request's input messages
    output_message_list: Optional[list[dict]] = None              # what the model answered
    model_response: Optional[ModelResponse] = None
    reward: Optional[float] = None
    parent: Optional["InteractionWithTokenLogpReward"] = None
    chat_template_type: str = "hf"                                # "hf" | "concat"
    created_at: float = field(default_factory=time.time)
    completion: Any = None
    api_type: str = "completion"                                  # "completion" | "response"
    _cache: Optional[dict] = None

    @property
    def has_tensor_data(self) -> bool:
        return self.model_response is not None

    @property
    def full_messages(self) -> list[dict]:
        return list(self.messages) + list(self.output_message_list or [])

    def to_tensor_dict(self) -> dict[str, torch.Tensor]:
        """``[1, L]`` tensors in the RLVR trajectory layout. With a parent (concat style) the
        parent's whole token sequence is the prefix: its generated tokens keep loss_mask 1
        and their original logprobs / versions, the tokens this call added to the prompt get
        loss_mask 0."""
        if self._cache is not None:
            return self._cache
        r = self.model_response
        assert r is not None, "interaction holds no token data"
        if self.parent is not None and self.chat_template_type == "concat":
            p = self.parent.to_tensor_dict()
            seq = p["input_ids"][0].tolist()
            lp = p["logprobs"][0].tolist()
            lm = p["loss_mask"][0].tolist()
            ver = p["versions"][0].tolist()
            plen = len(seq)
            if r.input_tokens[:plen] != seq:
                raise ValueError("concat export: the request's tokens do not extend its parent's sequence")
            extra = r.input_tokens[plen:]
        else:
            seq, lp, lm, ver = [], [], [], []
            extra = r.input_tokens
        seq += list(extra) + list(r.output_tokens)
        lp += [0.0] * len(extra) + list(r.output_logprobs)
        lm += [0] * len(extra) + [1] * r.output_len
        ver += [-1] * len(extra) + list(r.output_versions)
        L = len(seq)
        out = {
            "input_ids": torch.tensor(seq, dtype=torch.long).unsqueeze(0),
            "loss_mask": torch.tensor(lm, dtype=torch.int32).unsqueeze(0),
            "logprobs": torch.tensor(lp, dtype=torch.float32).unsqueeze(0),
            "versions": torch.tensor(ver, dtype=torch.int32).unsqueeze(0),
            "attention_mask": torch.ones(1, L, dtype=torch.bool),
            "rewards": torch.tensor([float(self.reward if self.reward is not None else 0.0)], dtype=torch.float32),
        }
        self._cache = out
        return out
