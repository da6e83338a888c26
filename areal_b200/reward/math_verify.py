"""Answer verification for math-style rewards without an external parser.

:class:`MathVerifyWorker` plays the role of the reference's worker around the ``math_verify`` package
(``areal/reward/__init__.py:15-117``): it pulls the final answer out of a response (``\\boxed{...}`` with
nested braces, ``#### x``, ``<answer>..</answer>``, ``[x]``, "the answer is x", else the last number),
turns both sides into a canonical value where it can (integers, decimals, thousands separators, percent,
``a/b``, ``\\frac{a}{b}``, ``\\sqrt{a}``, ``\\pi``, scientific notation, a leading currency sign or a
trailing unit word) and compares numerically after rounding to ``precision`` decimals, otherwise as normalised
strings (sets / tuples element-wise). A wall-clock limit guards the evaluation like the reference's.
The named dataset rewards of the reference sit on top: gsm8k, geometry3k (answer in square brackets),
clevr_count_70k (a count).
"""
from __future__ import annotations

import concurrent.futures
import math
import re
from fractions import Fraction
from typing import Optional

from ..utils import logging as alog

logger = alog.getLogger("math_verify")

_NUM_RE = re.compile(r"-?\d[\d,]*\.?\d*(?:[eE][-+]?\d+)?|-?\.\d+")


def last_boxed(text: str) -> Optional[str]:
    """Content of the last ``\\boxed{...}`` / ``\\fbox{...}`` with balanced braces."""
    best = None
    for m in re.finditer(r"\\(?:boxed|fbox)\s*\{", text):
        depth, i = 1, m.end()
        while i < len(text) and depth:
            depth += {"{": 1, "}": -1}.get(text[i], 0)
            i += 1
        if depth == 0:
            best = text[m.end():i - 1]
    return best


def extract_final_answer(text: str, try_extract_without_anchor: bool = True) -> Optional[str]:
    if text is None:
        return None
    text = str(text)
    b = last_boxed(text)
    if b is not None:
        return b.strip()
    m = re.findall(r"<answer>(.*?)</answer>", text, re.S)
    if m:
        return m[-1].strip()
    if "####" in text:
        return text.split("####")[-1].strip().splitlines()[0].strip() if text.split("####")[-1].strip() else None
    m = re.findall(r"(?:final answer|answer)\s*(?:is|:|=)\s*([^\n]+)", text, re.I)
    if m:
        return m[-1].strip().rstrip(".")
    if not try_extract_without_anchor:
        return None
    nums = _NUM_RE.findall(text)
    if nums:
        return nums[-1]
    return text.strip() or None


def _strip_latex(s: str) -> str:
    s = s.strip().strip("$").strip()
    s = re.sub(r"\\(?:left|right|displaystyle|,|;|!|quad|qquad)", "", s)
    s = re.sub(r"\\text\{([^{}]*)\}", r"\1", s)
    s = re.sub(r"\\mathrm\{([^{}]*)\}", r"\1", s)
    s = s.replace("\\%", "%").replace("\\$", "").replace("$", "")
    s = s.replace("\\dfrac", "\\frac").replace("\\tfrac", "\\frac")
    s = s.replace("^\\circ", "").replace("^{\\circ}", "").replace("°", "")
    return s.strip()


def _to_number(s: str) -> Optional[float]:
    """Numeric value of a normalised answer string, or None."""
    s = _strip_latex(s).rstrip(".")
    s = re.sub(r"^(?:usd|us\$|€|£)\s*", "", s, flags=re.I)
    pct = s.endswith("%")
    if pct:
        s = s[:-1].strip()
    # a trailing unit word ("12 cm", "5 apples")
    m = re.fullmatch(r"(.+?\d)\s*[a-zA-Z][a-zA-Z ./^0-9]*", s)
    if m and not re.search(r"\\|sqrt|pi", s):
        s = m.group(1)
    s = s.replace(",", "") if re.fullmatch(r"-?\d{1,3}(,\d{3})+(\.\d+)?", s) else s
    expr = s
    expr = re.sub(r"\\sqrt\s*\{([^{}]+)\}", r"sqrt(\1)", expr)
    expr = re.sub(r"\\sqrt\s*(\d+)", r"sqrt(\1)", expr)
    for _ in range(4):                       # innermost fractions first
        expr = re.sub(r"\\frac\s*\{([^{}]+)\}\s*\{([^{}]+)\}", r"((\1)/(\2))", expr)
    expr = expr.replace("\\pi", "pi").replace("\\cdot", "*").replace("\\times", "*").replace("^", "**")
    expr = re.sub(r"(\d)\s*(pi|sqrt)", r"\1*\2", expr)
    expr = re.sub(r"\)\s*(pi|sqrt|\()", r")*\1", expr)
    expr = expr.replace("{", "(").replace("}", ")")
    if not re.fullmatch(r"[\d\s+\-*/().eE]*(?:(?:pi|sqrt)[\d\s+\-*/().eE]*)*", expr) or not re.search(r"\d|pi", expr):
        return None
    try:
        v = eval(compile(expr, "<answer>", "eval"), {"__builtins__": {}}, {"pi": math.pi, "sqrt": math.sqrt})
    except Exception:
        return None
    if isinstance(v, complex) or not isinstance(v, (int, float)) or math.isnan(v) or math.isinf(v):
        return None
    return float(v) / 100.0 if pct else float(v)


def _norm_text(s: str) -> str:
    s = _strip_latex(s).lower().rstrip(".")
    s = re.sub(r"\s+", "", s)
    return s.replace("\\", "").replace("{", "").replace("}", "")


def _split_top(s: str) -> list[str]:
    """Top-level comma split of a tuple / set / interval body."""
    parts, depth, cur = [], 0, ""
    for ch in s:
        depth += ch in "({[" and 1 or (ch in ")}]" and -1 or 0)
        if ch == "," and depth == 0:
            parts.append(cur)
            cur = ""
        else:
            cur += ch
    return parts + [cur]


class MathVerifyWorker:
    def __init__(self, try_extract_without_anchor: bool = True, precision: int = 6, timeout: Optional[float] = 5.0):
        self.try_extract_without_anchor, self.precision, self.timeout = try_extract_without_anchor, precision, timeout

    def _equal(self, a: str, b: str) -> bool:
        x, y = _to_number(a), _to_number(b)
        if x is not None and y is not None:
            if x == y:
                return True
            # equal after rounding to ``precision`` decimals (the reference's float_rounding), or to 12 significant digits
            return round(x, self.precision) == round(y, self.precision) or abs(x - y) <= max(abs(x), abs(y)) * 1e-12
        sa, sb = _strip_latex(a), _strip_latex(b)
        if len(sa) > 1 and len(sb) > 1 and sa[0] in "([{" and sb[0] in "([{" and sa[0] == sb[0] and sa[-1] == sb[-1]:
            pa, pb = _split_top(sa[1:-1]), _split_top(sb[1:-1])
            if len(pa) == len(pb) and len(pa) > 1:
                if sa[0] == "{":           # a set: order does not matter
                    left = list(pb)
                    for e in pa:
                        hit = next((f for f in left if self._equal(e, f)), None)
                        if hit is None:
                            return False
                        left.remove(hit)
                    return True
                return all(self._equal(e, f) for e, f in zip(pa, pb))
        return _norm_text(a) == _norm_text(b) and _norm_text(a) != ""

    def _verify_impl(self, response: str, ground_truth: str) -> float:
        # a reference answer without an anchor is the answer itself ("\\frac{1}{2}", "(1, 2)"), not prose to search
        gold = extract_final_answer(ground_truth, False) or str(ground_truth).strip() or None
        pred = extract_final_answer(response, self.try_extract_without_anchor)
        if gold is None or pred is None:
            return 0.0
        return 1.0 if self._equal(pred, gold) else 0.0

    def verify(self, response: str, ground_truth: str) -> float:
        try:
            if self.timeout is None:
                return self._verify_impl(response, ground_truth)
            with concurrent.futures.ThreadPoolExecutor(max_workers=1) as ex:
                return ex.submit(self._verify_impl, str(response), str(ground_truth)).result(timeout=self.timeout)
        except concurrent.futures.TimeoutError:
            logger.warning("verification timed out after %.1fs", self.timeout)
            return 0.0
        except Exception:
            logger.warning("verification failed", exc_info=True)
            return 0.0


_WORKER: Optional[MathVerifyWorker] = None


def get_math_verify_worker() -> MathVerifyWorker:
    global _WORKER
    if _WORKER is None:
        _WORKER = MathVerifyWorker()
    return _WORKER


def math_verify_reward_fn(prompt, completions, prompt_ids, completion_ids, answer=None, **kwargs) -> float:
    return get_math_verify_worker().verify(str(completions or ""), str(answer))


def _bracket_or_last_number(text: str) -> str:
    m = re.findall(r"\[([^\]]+)\]", text)
    if m:
        return m[-1]
    nums = re.findall(r"-?\d*\.?\d+", text.replace(",", ""))
    return nums[-1] if nums else ""


def geometry3k_reward_fn(prompt, completions, prompt_ids, completion_ids, answer=None, **kwargs) -> float:
    """The response names its answer in square brackets (else its last number counts); compared with the verifier
    (reference ``areal/reward/geometry3k.py``)."""
    sol = _bracket_or_last_number(str(completions or ""))
    ans = _bracket_or_last_number(str(answer)) or str(answer)
    if not sol or not ans:
        return 0.0
    return get_math_verify_worker().verify(sol, ans)


def clevr_count_70k_reward_fn(prompt, completions, prompt_ids, completion_ids, answer=None, **kwargs) -> float:
    """Object counting: the bracketed (else last) number of the response must equal the count (reference
    ``areal/reward/clevr_count_70k.py``)."""
    sol = _bracket_or_last_number(str(completions or ""))
    ans = _bracket_or_last_number(str(answer)) or str(answer)
    try:
        return 1.0 if sol and ans and float(sol) == float(ans) else 0.0
    except ValueError:
        return 0.0
