"""Writes ``docs/config_reference.md`` from the configuration dataclasses of ``areal_b200/api/cli_args.py``.

    python -m areal_b200.tools.generate_cli_docs            # rewrite the file
    python -m areal_b200.tools.generate_cli_docs --check    # exit 1 when the committed file is out of date

One section per dataclass (alphabetical), one table row per field with its type and default; the trailing comment
of a field's line in the source becomes its note; a field whose name occurs nowhere else in the package is marked as
accepted for compatibility only. Reference: ``docs/generate_cli_docs.py`` of the reference, which
renders its ``cli_args.py`` the same way."""
from __future__ import annotations

import argparse
import dataclasses
import inspect
import os
import re
import sys
import typing

HEAD = ("# Configuration reference\n\nGenerated from `areal_b200/api/cli_args.py` by `python -m areal_b200.tools.generate_cli_docs`. Every YAML key maps to a "
        "dataclass field; unknown keys are rejected (backend-specific sections `sglang`, `vllm`, `megatron`, `archon` keep unknown keys in `extra`).\n\n")


def _type_name(t) -> str:
    if isinstance(t, str):
        return t
    origin = typing.get_origin(t)
    if origin is typing.Union:
        args = [a for a in typing.get_args(t)]
        if len(args) == 2 and type(None) in args:
            other = args[0] if args[1] is type(None) else args[1]
            return f"Optional[{_type_name(other)}]"
        return " | ".join(_type_name(a) for a in args)
    if origin is not None:
        inner = ", ".join(_type_name(a) for a in typing.get_args(t))
        name = getattr(origin, "__name__", str(origin))
        return f"{name}[{inner}]" if inner else name
    return getattr(t, "__name__", str(t))


def _default(f: dataclasses.Field) -> str:
    if f.default is not dataclasses.MISSING:
        v = repr(f.default)
    elif f.default_factory is not dataclasses.MISSING:      # type: ignore[misc]
        try:
            v = repr(f.default_factory())                   # type: ignore[misc]
        except Exception:
            v = "<factory>"
    else:
        return "required"
    return v if len(v) <= 60 else v[:57] + "..."


def _notes(cls) -> dict[str, str]:
    """Field name -> trailing ``# comment`` of its line in the class body."""
    out = {}
    try:
        src = inspect.getsource(cls)
    except (OSError, TypeError):
        return out
    for line in src.splitlines():
        m = re.match(r"\s+(\w+)\s*:\s*[^#]+#\s*(.+)$", line)
        if m:
            out[m.group(1)] = m.group(2).strip().replace("|", "\\|")
    return out


COMPAT_NOTE = "accepted so that configuration files of the reference load unchanged; not read by this implementation"


def _package_text() -> str:
    """All source text of the package (and the benchmark entry point) except the configuration module itself."""
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    chunks = []
    for dp, dns, fs in os.walk(root):
        dns[:] = sorted(d for d in dns if d != "__pycache__")
        for f in sorted(fs):
            if f.endswith(".py") and not (dp.endswith(os.sep + "api") and f == "cli_args.py"):
                with open(os.path.join(dp, f)) as fh:
                    chunks.append(fh.read())
    bench = os.path.join(os.path.dirname(root), "bench.py")
    if os.path.exists(bench):
        with open(bench) as fh:
            chunks.append(fh.read())
    for dp, dns, fs in os.walk(os.path.join(os.path.dirname(root), "examples")):      # example scripts read config fields too
        dns[:] = sorted(d for d in dns if d != "__pycache__")
        for f in sorted(fs):
            if f.endswith(".py"):
                with open(os.path.join(dp, f)) as fh:
                    chunks.append(fh.read())
    return "\n".join(chunks)


def render() -> str:
    from ..api import cli_args as C

    text = _package_text()
    used_cache: dict[str, bool] = {}

    def used(name: str) -> bool:
        if name not in used_cache:
            used_cache[name] = re.search(r"\b%s\b" % re.escape(name), text) is not None
        return used_cache[name]

    classes = sorted((c for _, c in inspect.getmembers(C, inspect.isclass)
                      if dataclasses.is_dataclass(c) and c.__module__ == C.__name__ and not c.__name__.startswith("_")),
                     key=lambda c: c.__name__)
    parts = [HEAD]
    for cls in classes:
        parts.append(f"\n## {cls.__name__}\n\n")
        doc = inspect.getdoc(cls)
        if doc and not doc.startswith(cls.__name__ + "("):
            parts.append(doc.split("\n\n")[0].replace("\n", " ") + "\n\n")
        notes = _notes(cls)
        hints = {}
        try:
            hints = typing.get_type_hints(cls)
        except Exception:
            pass
        parts.append("| field | type | default | note |\n|---|---|---|---|\n")
        passthrough = cls.__name__ in ("SGLangConfig", "vLLMConfig")       # every field becomes a flag of the external server's command line
        for f in dataclasses.fields(cls):
            note = notes.get(f.name, "")
            if not passthrough and not dataclasses.is_dataclass(f.type) and not used(f.name):
                note = (note + "; " if note else "") + COMPAT_NOTE
            parts.append(f"| `{f.name}` | `{_type_name(hints.get(f.name, f.type))}` | `{_default(f)}` | {note} |\n")
    return "".join(parts)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--check", action="store_true")
    ap.add_argument("--out", default=os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "docs", "config_reference.md"))
    a = ap.parse_args(argv)
    text = render()
    if a.check:
        try:
            with open(a.out) as f:
                same = f.read() == text
        except OSError:
            same = False
        if not same:
            print(f"{a.out} is out of date: run python -m areal_b200.tools.generate_cli_docs")
        return 0 if same else 1
    with open(a.out, "w") as f:
        f.write(text)
    print(f"wrote {a.out} ({text.count(chr(10))} lines)")
    return 0


if __name__ == "__main__":
    sys.exit(main())
