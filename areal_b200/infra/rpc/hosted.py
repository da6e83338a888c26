"""Engines hosted by this process, by name. Lets an engine that is created later (an OpenAI-compatible proxy over
the rollout engine of the same worker) find the one it fronts. A module of its own: the RPC server usually runs
as ``__main__``, so a registry inside it would exist twice."""
from __future__ import annotations

from typing import Any

HOSTED_ENGINES: dict[str, Any] = {}
