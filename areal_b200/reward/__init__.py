"""Reward functions (reference: ``areal/reward/*``): exact-match math answers with a light
normaliser (no external verifier needed), plus the synthetic rewards used by benchmarks."""
from __future__ import annotations

import re
from typing import Optional

from ..dataset import arithmetic_reward_fn, bernoulli_reward_fn  # noqa: F401

_BOXED = re.compile(r"\\boxed\{([^{}]*)\}")
_NUM = re.compile(r"-?\d[\d,]*\.?\d*")


def extract_answer(text: str) -> Optional[str]:
    if text is None:
        return None
    m = _BOXED.findall(text)
    if m:
        return m[-1].strip()
    if "####" in text:
        return text.split("####")[-1].strip()
    nums = _NUM.findall(text)
    return nums[-1] if nums else None


def _norm(s: Optional[str]) -> Optional[str]:
    if s is None:
        return None
    s = s.replace(",", "").replace("$", "").strip().rstrip(".")
    try:
        f = float(s)
        return str(int(f)) if f == int(f) else repr(f)
    except ValueError:
        return s.lower()


def gsm8k_reward_fn(prompt, completions, prompt_ids, completion_ids, answer=None, **kwargs) -> float:
    gold = _norm(extract_answer(str(answer)))
    pred = _norm(extract_answer(completions or ""))
    return 1.0 if gold is not None and pred == gold else 0.0


math_verify_reward_fn = gsm8k_reward_fn
