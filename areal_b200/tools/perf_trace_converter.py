"""Merges per-rank ``traces-r*.jsonl`` files (and rollout ``sessions.jsonl``) into one Chrome
/ Perfetto trace (``chrome://tracing`` JSON object format).

    python -m areal_b200.tools.perf_trace_converter <dir-or-files...> -o trace.json [--sessions]

Ranks become processes (with name metadata), threads keep their ids, timestamps are aligned
to the earliest event. Session phases are rendered as one track per rollout session.
Reference: ``areal/tools/perf_trace_converter.py``."""
from __future__ import annotations

import argparse
import glob
import json
import os
import sys
from typing import Iterable


def _read_jsonl(path: str) -> Iterable[dict]:
    with open(path) as f:
        for ln, line in enumerate(f, 1):
            line = line.strip()
            if not line:
                continue
            try:
                yield json.loads(line)
            except json.JSONDecodeError:
                print(f"warning: {path}:{ln}: not JSON, skipped", file=sys.stderr)


def collect_files(inputs: list[str]) -> tuple[list[str], list[str]]:
    traces, sessions = [], []
    for p in inputs:
        if os.path.isdir(p):
            traces += sorted(glob.glob(os.path.join(p, "**", "traces-r*.jsonl"), recursive=True))
            sessions += sorted(glob.glob(os.path.join(p, "**", "sessions.jsonl"), recursive=True))
        elif os.path.basename(p).startswith("sessions"):
            sessions.append(p)
        else:
            traces.append(p)
    return traces, sessions


def convert(trace_files: list[str], session_files: list[str] = (), align: bool = True) -> dict:
    events: list[dict] = []
    pids = set()
    for f in trace_files:
        for e in _read_jsonl(f):
            if "ph" not in e or "ts" not in e:
                continue
            events.append(e)
            pids.add(e.get("pid", 0))
    t_min = min((e["ts"] for e in events), default=0.0) if align else 0.0
    for e in events:
        e["ts"] = e["ts"] - t_min
    meta = [{"name": "process_name", "ph": "M", "pid": p, "tid": 0, "args": {"name": f"rank {p}"}} for p in sorted(pids)]
    sess_pid = (max(pids) + 1) if pids else 0
    n_sess = 0
    s_min = None
    sess = [s for f in session_files for s in _read_jsonl(f)]
    if sess:
        s_min = min(s.get("submit_ts", 0.0) for s in sess)
        meta.append({"name": "process_name", "ph": "M", "pid": sess_pid, "tid": 0, "args": {"name": "rollout sessions"}})
    for s in sess:
        tid = int(s.get("session_id", n_sess))
        n_sess += 1
        for ph in s.get("phases", []):
            events.append({"name": ph["name"], "cat": "session", "ph": "X", "ts": (ph["start"] - s_min) * 1e6,
                           "dur": max(0.0, ph["end"] - ph["start"]) * 1e6, "pid": sess_pid, "tid": tid,
                           "args": {"task_id": s.get("task_id"), "status": s.get("status"), "rank": s.get("rank")}})
    events.sort(key=lambda e: (e.get("pid", 0), e["ts"]))
    return {"traceEvents": meta + events, "displayTimeUnit": "ms",
            "otherData": {"ranks": sorted(pids), "sessions": n_sess, "source_files": len(trace_files) + len(session_files)}}


def summarize(trace: dict) -> dict[str, dict]:
    """Total / mean duration per event name (complete events only)."""
    out: dict[str, dict] = {}
    for e in trace["traceEvents"]:
        if e.get("ph") != "X":
            continue
        d = out.setdefault(e["name"], {"count": 0, "total_ms": 0.0})
        d["count"] += 1
        d["total_ms"] += e.get("dur", 0.0) / 1e3
    for d in out.values():
        d["mean_ms"] = d["total_ms"] / d["count"]
    return out


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("inputs", nargs="+")
    ap.add_argument("-o", "--output", default="trace.json")
    ap.add_argument("--no-align", action="store_true")
    ap.add_argument("--summary", action="store_true", help="print per-scope totals")
    a = ap.parse_args(argv)
    tr, se = collect_files(a.inputs)
    if not tr and not se:
        ap.error("no trace files found")
    trace = convert(tr, se, align=not a.no_align)
    with open(a.output, "w") as f:
        json.dump(trace, f)
    print(f"wrote {a.output}: {len(trace['traceEvents'])} events from {len(tr)} trace and {len(se)} session files")
    if a.summary:
        for name, d in sorted(summarize(trace).items(), key=lambda kv: -kv[1]["total_ms"]):
            print(f"{name:40s} n={d['count']:6d} total={d['total_ms']:10.2f} ms mean={d['mean_ms']:8.3f} ms")


if __name__ == "__main__":
    main()
