"""Timeline of rollout sessions from ``sessions.jsonl`` (written by the session tracer): one row per
session, one coloured bar per phase (generate / reward / tool call / ...), plus a text summary with
per-phase totals, the time sessions spent outside any phase, and the distribution of session lengths.
The figure is a self-contained SVG or HTML file (no plotting library needed).

    python -m areal_b200.tools.plot_session_trace <trace dir or sessions.jsonl ...> -o sessions.html [--max-sessions 400]

Reference: ``areal/tools/plot_session_trace.py`` (Plotly figure of the same records)."""
from __future__ import annotations

import argparse
import glob
import html
import json
import os
import sys
from collections import defaultdict

PALETTE = ["#4e79a7", "#f28e2b", "#59a14f", "#e15759", "#b07aa1", "#76b7b2", "#edc948", "#ff9da7", "#9c755f", "#bab0ac"]


def load_sessions(paths: list[str]) -> list[dict]:
    files: list[str] = []
    for p in paths:
        if os.path.isdir(p):
            files += sorted(glob.glob(os.path.join(p, "**", "sessions.jsonl"), recursive=True))
        else:
            files.append(p)
    out = []
    for fn in files:
        with open(fn) as f:
            for line in f:
                line = line.strip()
                if line:
                    out.append(json.loads(line))
    out.sort(key=lambda s: s.get("submit_ts", 0.0))
    return out


def summarize(sessions: list[dict]) -> dict:
    """Per-phase totals and session statistics (seconds)."""
    phase_tot: dict[str, float] = defaultdict(float)
    phase_cnt: dict[str, int] = defaultdict(int)
    durs, idle, status = [], [], defaultdict(int)
    for s in sessions:
        t0, t1 = s.get("submit_ts", 0.0), s.get("end_ts", s.get("submit_ts", 0.0))
        busy = 0.0
        for ph in s.get("phases", []):
            d = max(0.0, ph["end"] - ph["start"])
            phase_tot[ph["name"]] += d
            phase_cnt[ph["name"]] += 1
            busy += d
        durs.append(max(0.0, t1 - t0))
        idle.append(max(0.0, (t1 - t0) - busy))
        status[s.get("status", "?")] += 1
    durs_sorted = sorted(durs)

    def pct(q):
        return durs_sorted[min(len(durs_sorted) - 1, int(q * len(durs_sorted)))] if durs_sorted else 0.0
    return dict(n_sessions=len(sessions), status=dict(status), phase_seconds=dict(phase_tot), phase_counts=dict(phase_cnt),
                session_seconds=dict(mean=sum(durs) / len(durs) if durs else 0.0, p50=pct(0.5), p90=pct(0.9), p99=pct(0.99), max=max(durs, default=0.0)),
                unattributed_seconds=sum(idle))


def render_svg(sessions: list[dict], max_sessions: int = 400, width: int = 1200, row_h: int = 6) -> str:
    sessions = sessions[:max_sessions]
    if not sessions:
        return '<svg xmlns="http://www.w3.org/2000/svg" width="200" height="40"><text x="5" y="20">no sessions</text></svg>'
    t0 = min(s.get("submit_ts", 0.0) for s in sessions)
    t1 = max(s.get("end_ts", s.get("submit_ts", 0.0)) for s in sessions)
    span = max(1e-9, t1 - t0)
    names = sorted({ph["name"] for s in sessions for ph in s.get("phases", [])})
    color = {n: PALETTE[i % len(PALETTE)] for i, n in enumerate(names)}
    left, top = 60, 30 + 14 * ((len(names) + 5) // 6)
    H = top + row_h * len(sessions) + 30
    x = lambda t: left + (t - t0) / span * (width - left - 10)
    out = [f'<svg xmlns="http://www.w3.org/2000/svg" width="{width}" height="{H}" font-family="monospace" font-size="10">']
    for i, n in enumerate(names):                                   # legend
        lx, ly = left + (i % 6) * 180, 12 + 14 * (i // 6)
        out.append(f'<rect x="{lx}" y="{ly - 8}" width="10" height="10" fill="{color[n]}"/><text x="{lx + 14}" y="{ly + 1}">{html.escape(n)}</text>')
    for k in range(6):                                               # time axis
        t = t0 + span * k / 5
        out.append(f'<line x1="{x(t):.1f}" y1="{top - 4}" x2="{x(t):.1f}" y2="{H - 24}" stroke="#ddd"/>'
                   f'<text x="{x(t) - 10:.1f}" y="{H - 10}">{t - t0:.1f}s</text>')
    for r, s in enumerate(sessions):
        y = top + r * row_h
        a, b = s.get("submit_ts", t0), s.get("end_ts", s.get("submit_ts", t0))
        ok = s.get("status") in ("accepted", "ok", "done", "finished")
        out.append(f'<rect x="{x(a):.1f}" y="{y}" width="{max(0.5, x(b) - x(a)):.1f}" height="{row_h - 1}" fill="{"#eee" if ok else "#fdd"}"/>')
        for ph in s.get("phases", []):
            out.append(f'<rect x="{x(ph["start"]):.1f}" y="{y}" width="{max(0.5, x(ph["end"]) - x(ph["start"])):.1f}" height="{row_h - 1}" '
                       f'fill="{color[ph["name"]]}"><title>session {s.get("session_id")} {html.escape(ph["name"])} '
                       f'{ph["end"] - ph["start"]:.3f}s</title></rect>')
    out.append(f'<text x="2" y="{top + 8}">sessions</text></svg>')
    return "\n".join(out)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("paths", nargs="+")
    ap.add_argument("-o", "--output", default="sessions.html")
    ap.add_argument("--max-sessions", type=int, default=400)
    a = ap.parse_args(argv)
    sessions = load_sessions(a.paths)
    summ = summarize(sessions)
    svg = render_svg(sessions, a.max_sessions)
    if a.output.endswith(".svg"):
        body = svg
    else:
        body = ("<html><body><h3>rollout sessions</h3><pre>" + html.escape(json.dumps(summ, indent=2)) + "</pre>" + svg + "</body></html>")
    with open(a.output, "w") as f:
        f.write(body)
    print(json.dumps(summ))
    return 0


if __name__ == "__main__":
    sys.exit(main())
