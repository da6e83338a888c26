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


from .math_verify import (MathVerifyWorker, clevr_count_70k_reward_fn, extract_final_answer, geometry3k_reward_fn,  # noqa: E402,F401
                          get_math_verify_worker, math_verify_reward_fn)


def countdown_reward_fn(prompt, completions, prompt_ids, completion_ids, numbers=None, target=None, **kwargs) -> float:
    """Countdown: the completion's last equation (``<answer>...</answer>`` if present, else the last
    line with digits) must use exactly the given numbers once each with + - * / and evaluate to
    ``target``. 1.0 for a correct equation, 0.1 for a well-formed one with the wrong value, else 0."""
    import ast
    import re

    text = completions or ""
    m = re.findall(r"<answer>(.*?)</answer>", text, re.S)
    expr = m[-1] if m else next((l for l in reversed(text.strip().splitlines()) if re.search(r"\d", l)), "")
    expr = expr.split("=")[0].strip()
    if not expr or not re.fullmatch(r"[\d\s+\-*/().]+", expr):
        return 0.0
    used = sorted(int(x) for x in re.findall(r"\d+", expr))
    if numbers is None or used != sorted(int(x) for x in numbers):
        return 0.0
    try:
        tree = ast.parse(expr, mode="eval")
        ok_nodes = (ast.Expression, ast.BinOp, ast.UnaryOp, ast.Constant, ast.Add, ast.Sub, ast.Mult, ast.Div, ast.USub)
        if not all(isinstance(n, ok_nodes) for n in ast.walk(tree)):
            return 0.0
        val = eval(compile(tree, "<countdown>", "eval"), {"__builtins__": {}}, {})
    except Exception:
        return 0.0
    return 1.0 if target is not None and abs(val - float(target)) < 1e-6 else 0.1
