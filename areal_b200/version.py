"""Package version and the state of the source tree it runs from (commit, branch, uncommitted changes), read once.

Reference: ``areal/version.py`` (version + git info stamped into experiment metadata).
"""
from __future__ import annotations

import os
import subprocess
from dataclasses import dataclass

__version__ = "0.2.0"


@dataclass(frozen=True)
class VersionInfo:
    version: str
    commit: str = "unknown"
    branch: str = "unknown"
    is_dirty: bool = False

    @property
    def full_version(self) -> str:
        return f"{self.version}+{self.commit[:8]}" if self.commit != "unknown" else self.version

    @property
    def full_version_with_dirty_description(self) -> str:
        return self.full_version + (".dirty" if self.is_dirty else "")


def _git(*args: str) -> str:
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    try:
        return subprocess.run(["git", "-C", root, *args], capture_output=True, text=True, timeout=5, check=True).stdout.strip()
    except Exception:  # noqa: BLE001  (no git, not a checkout, a sandbox without subprocesses: the version alone)
        return ""


def _read() -> VersionInfo:
    commit = _git("rev-parse", "HEAD")
    if not commit:
        return VersionInfo(__version__)
    return VersionInfo(__version__, commit, _git("rev-parse", "--abbrev-ref", "HEAD") or "unknown", bool(_git("status", "--porcelain", "--untracked-files=no")))


class _Lazy:
    """``version_info.commit`` etc.; git is asked on first use, not at import."""

    _v = None

    def __getattr__(self, name):
        if _Lazy._v is None:
            _Lazy._v = _read()
        return getattr(_Lazy._v, name)


version_info = _Lazy()
