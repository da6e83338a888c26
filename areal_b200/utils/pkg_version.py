"""Package presence / version checks (reference: ``areal/utils/pkg_version.py``)."""
from __future__ import annotations

import importlib.metadata
import importlib.util


def is_available(pkg: str) -> bool:
    return importlib.util.find_spec(pkg) is not None


def get_version(pkg: str) -> str | None:
    try:
        return importlib.metadata.version(pkg)
    except importlib.metadata.PackageNotFoundError:
        return None


def _key(v: str) -> tuple:
    out = []
    for part in v.split("+")[0].split("."):
        digits = "".join(ch for ch in part if ch.isdigit())
        out.append(int(digits) if digits else 0)
    return tuple(out)


def is_version_greater_or_equal(pkg: str, target: str) -> bool:
    v = get_version(pkg)
    return v is not None and _key(v) >= _key(target)


def is_version_less(pkg: str, target: str) -> bool:
    v = get_version(pkg)
    return v is not None and _key(v) < _key(target)
