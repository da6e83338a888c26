"""Per-episode store of model calls with reward assignment and export. Reference:
``areal/experimental/openai/cache.py`` (``InteractionCache`` :39, ``apply_reward_discount``
:208, parent linking in ``__setitem__`` :260, ``export_interactions`` :403)."""
from __future__ import annotations

from collections import OrderedDict
from typing import Callable, Optional

from ..utils import logging as alog
from .types import InteractionWithTokenLogpReward

logger = alog.getLogger("openai_cache")


def _norm_msg(m: dict) -> tuple:
    c = m.get("content")
    if isinstance(c, list):  # content parts
        c = "".join(p.get("text", "") if isinstance(p, dict) else str(p) for p in c)
    tc = m.get("tool_calls") or None
    tcs = tuple((t.get("function", {}).get("name"), t.get("function", {}).get("arguments")) for t in tc) if tc else None
    return (m.get("role"), c or "", tcs, m.get("tool_call_id"))


def default_prefix_matcher(a: list[dict], b: list[dict]) -> bool:
    """True when message list ``a`` is a strict prefix of ``b``."""
    if len(a) >= len(b):
        return False
    return all(_norm_msg(x) == _norm_msg(y) for x, y in zip(a, b))


class InteractionCache(OrderedDict):
    def __init__(self, prefix_matcher: Callable[[list[dict], list[dict]], bool] = default_prefix_matcher):
        super().__init__()
        self._matcher = prefix_matcher
        self._discount_applied = False

    # ---- rewards
    @property
    def last_interaction_id(self) -> str:
        return next(reversed(self))

    @property
    def total_reward(self) -> float:
        return sum(i.reward or 0.0 for i in self.values())

    def set_reward(self, interaction_id: str, reward: float) -> None:
        self[interaction_id].reward = float(reward)
        self[interaction_id]._cache = None

    def set_last_reward(self, reward: float) -> None:
        self.set_reward(self.last_interaction_id, reward)

    def apply_reward_discount(self, turn_discount: float = 1.0) -> dict:
        """Walks the calls newest → oldest: ``reward[i] += turn_discount * reward[i+1]``
        (unset rewards count as 0). May run once per episode."""
        if self._discount_applied:
            raise RuntimeError("apply_reward_discount should only be called once")
        self._discount_applied = True
        running = 0.0
        for k, it in enumerate(reversed(list(self.values()))):
            if it.reward is None:
                if k == 0:
                    logger.warning("the most recent interaction has no reward; using 0")
                it.reward = 0.0
            running = running * turn_discount + it.reward
            it.reward = running
            it._cache = None
        return dict(self)

    # ---- tree
    def __setitem__(self, key: str, value: InteractionWithTokenLogpReward) -> None:
        """Links ``value`` to the cached call whose full conversation (input + answer) is the
        longest strict prefix of ``value``'s input messages."""
        if key not in self and value.parent is None and value.chat_template_type == "concat":
            best, best_len = None, -1
            for other in self.values():
                if other.output_message_list is None:
                    continue
                fm = other.full_messages
                if len(fm) > best_len and self._matcher(fm, value.messages + [{}]) and len(fm) <= len(value.messages):
                    best, best_len = other, len(fm)
            value.parent = best
        super().__setitem__(key, value)

    def export_interactions(self, style: str = "concat", reward_discount: Optional[float] = None) -> dict:
        """``individual``: every completed call. ``concat``: only the leaves of the
        conversation tree (each carries its ancestors' tokens as prefix)."""
        if reward_discount is not None and not self._discount_applied:
            self.apply_reward_discount(reward_discount)
        done = {k: v for k, v in self.items() if v.interaction_id is not None and v.output_message_list is not None}
        if not done:
            return {}
        if style == "individual":
            return done
        if style == "concat":
            for v in done.values():
                if v.chat_template_type != "concat":
                    raise ValueError("'concat' export needs chat_template_type='concat' on every interaction: a chat "
                                     "template may add or drop tokens between turns; use 'individual' instead")
            parents = {id(v.parent) for v in done.values() if v.parent is not None}
            return {k: v for k, v in done.items() if id(v) not in parents}
        raise ValueError(f"invalid export style {style!r}")
