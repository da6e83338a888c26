"""Per-episode context (is_eval, task id, sample index) carried through asyncio via
``contextvars`` (reference: ``areal/infra/workflow_context.py:25-60``)."""
from __future__ import annotations

import contextvars
from contextlib import contextmanager
from dataclasses import dataclass
from typing import Optional


@dataclass(frozen=True)
class WorkflowContext:
    is_eval: bool = False
    task_id: Optional[int] = None
    sample_idx: Optional[int] = None


_CTX: contextvars.ContextVar[WorkflowContext] = contextvars.ContextVar("areal_workflow_ctx", default=WorkflowContext())


def get() -> WorkflowContext:
    return _CTX.get()


@contextmanager
def scoped(is_eval: bool = False, task_id: Optional[int] = None, sample_idx: Optional[int] = None):
    tok = _CTX.set(WorkflowContext(is_eval, task_id, sample_idx))
    try:
        yield
    finally:
        _CTX.reset(tok)


def stat_scope() -> str:
    return "eval-rollout" if get().is_eval else "rollout"
