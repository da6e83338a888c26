"""``import_from_string("pkg.mod.attr")`` / ``"pkg.mod:attr"`` helper
(reference: ``areal/utils/dynamic_import.py``)."""
from __future__ import annotations

import importlib


def import_from_string(path: str):
    if not isinstance(path, str) or not path:
        raise ValueError("import path must be a non-empty string")
    if ":" in path:
        mod, _, attr = path.partition(":")
    else:
        mod, _, attr = path.rpartition(".")
    if not mod or not attr:
        raise ValueError(f"'{path}' is not a dotted import path")
    m = importlib.import_module(mod)
    obj = m
    for part in attr.split("."):
        obj = getattr(obj, part)
    return obj
