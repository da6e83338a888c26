"""Run-mode switches read from the environment (reference: ``areal/utils/environ.py``)."""
from __future__ import annotations

import os


def _flag(name: str, default: str = "0") -> bool:
    return os.environ.get(name, default).lower() in ("1", "true", "yes", "on")


def is_single_controller() -> bool:
    """True when this process is the controller of RPC workers (no torchrun environment)."""
    if "AREAL_SPMD_MODE" in os.environ:
        return not _flag("AREAL_SPMD_MODE")
    return "RANK" not in os.environ and "WORLD_SIZE" not in os.environ


def is_recover_run() -> bool:
    return _flag("AREAL_RECOVER_RUN")


def force_cpu() -> bool:
    return _flag("AREAL_FORCE_CPU")


def in_ci() -> bool:
    return _flag("CI") or _flag("AREAL_IS_IN_CI")


def llm_server_addrs() -> list[str]:
    v = os.environ.get("AREAL_LLM_SERVER_ADDRS", "")
    return [a for a in v.split(",") if a]
