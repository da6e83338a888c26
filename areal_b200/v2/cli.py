"""``python -m areal_b200.v2.cli <service> <action>``: start / inspect services from the shell;
started services are recorded in a state file so later invocations find them. Reference:
``areal/v2/cli/*`` (``areal inference ...``, ``areal agent ...`` with persisted state).

    inference serve  --model-path P [--preset NAME] [--port N]      rollout server (HTTP)
    inference status                                                 health of recorded servers
    weight-update serve [--port N]                                   weight-update gateway
    state show | state clear
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading

from .common import HTTPError, call

STATE = os.environ.get("AREAL_V2_STATE", os.path.join(os.path.expanduser("~"), ".areal_b200", "v2_state.json"))


def load_state() -> dict:
    try:
        with open(STATE) as f:
            return json.load(f)
    except (OSError, json.JSONDecodeError):
        return {"services": []}


def save_state(st: dict) -> None:
    os.makedirs(os.path.dirname(STATE), exist_ok=True)
    tmp = STATE + ".tmp"
    with open(tmp, "w") as f:
        json.dump(st, f, indent=1)
    os.replace(tmp, STATE)


def record(kind: str, address: str, **extra) -> None:
    st = load_state()
    st["services"] = [s for s in st["services"] if s["address"] != address] + [dict(kind=kind, address=address, pid=os.getpid(), **extra)]
    save_state(st)


def cmd_status(kind: str) -> int:
    rc = 0
    for s in load_state()["services"]:
        if kind and s["kind"] != kind:
            continue
        try:
            h = call(f"http://{s['address']}/health", timeout=3)
            print(f"{s['kind']:16s} {s['address']:22s} ok   {json.dumps(h)[:100]}")
        except HTTPError as e:
            rc = 1
            print(f"{s['kind']:16s} {s['address']:22s} DOWN {e.message[:80]}")
    return rc


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="areal_b200.v2.cli")
    sub = ap.add_subparsers(dest="service", required=True)
    inf = sub.add_parser("inference")
    inf.add_argument("action", choices=["serve", "status"])
    inf.add_argument("--model-path", default="")
    inf.add_argument("--preset", default="")
    inf.add_argument("--port", type=int, default=0)
    inf.add_argument("--host", default="127.0.0.1")
    wu = sub.add_parser("weight-update")
    wu.add_argument("action", choices=["serve", "status"])
    wu.add_argument("--port", type=int, default=0)
    wu.add_argument("--host", default="127.0.0.1")
    stp = sub.add_parser("state")
    stp.add_argument("action", choices=["show", "clear"])
    a = ap.parse_args(argv)
    if a.service == "state":
        if a.action == "clear":
            save_state({"services": []})
        print(json.dumps(load_state(), indent=1))
        return 0
    if a.action == "status":
        return cmd_status("inference" if a.service == "inference" else "weight-update")
    if a.service == "inference":
        from ..engine import server

        args = ["--host", a.host] + (["--port", str(a.port)] if a.port else []) + (["--model-path", a.model_path] if a.model_path else []) + \
            (["--preset", a.preset] if a.preset else [])
        threading.Timer(0.0, lambda: None).start()
        # the server prints its address; record it once known
        orig_print = print

        def hooked(*p, **k):
            if p and isinstance(p[0], str) and p[0].startswith("INFER_SERVER_READY"):
                record("inference", p[0].split()[1], model_path=a.model_path, preset=a.preset)
            orig_print(*p, **k)
        server.print = hooked  # type: ignore[attr-defined]
        server.main(args)
        return 0
    from .weight_update.gateway import WeightUpdateGateway

    gw = WeightUpdateGateway(a.host, a.port or None).start()
    record("weight-update", gw.address)
    print(f"WEIGHT_UPDATE_GATEWAY_READY {gw.address}", flush=True)
    try:
        threading.Event().wait()
    except KeyboardInterrupt:
        pass
    gw.stop()
    return 0


if __name__ == "__main__":
    sys.exit(main())
