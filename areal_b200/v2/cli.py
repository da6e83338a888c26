"""``python -m areal_b200.v2.cli <service> <action>``: start / inspect services from the shell;
started services are recorded in a state file so later invocations find them. Reference:
``areal/v2/cli/*`` (``areal inference ...``, ``areal agent ...`` with persisted state).

    inference serve  --model-path P [--preset NAME] [--port N]      rollout server (HTTP)
    inference status | ps | models | stop [--address A]             health, table, model list, stop by recorded pid
    weight-update serve [--port N] | status                         weight-update gateway
    data serve worker|router|gateway [--router A] [--admin-key K]   one role of the data service
    sandbox serve [--port N] [--api-key K]                          code-execution server
    training run SCRIPT --config FILE [overrides ...]               an experiment through the local launcher
    logs NAME [-n LINES]                                             tail of a recorded service's log file
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


def cmd_ps(kind: str) -> int:
    rows = [s for s in load_state()["services"] if not kind or s["kind"] == kind]
    print(f"{'KIND':16s} {'ADDRESS':22s} {'PID':>8s}  ALIVE  EXTRA")
    for s in rows:
        alive = _pid_alive(int(s.get("pid", 0)))
        extra = {k: v for k, v in s.items() if k not in ("kind", "address", "pid") and v}
        print(f"{s['kind']:16s} {s['address']:22s} {s.get('pid', 0):8d}  {'yes' if alive else 'no ':5s}  {json.dumps(extra)[:80]}")
    return 0


def _pid_alive(pid: int) -> bool:
    if pid <= 0:
        return False
    try:
        os.kill(pid, 0)
        return True
    except (ProcessLookupError, PermissionError):
        return False


def cmd_stop(kind: str, address: str = "") -> int:
    """Ends recorded services of ``kind`` (one address, or all) by the exact pid they recorded, and drops them
    from the state file."""
    import signal

    st = load_state()
    keep, n = [], 0
    for s in st["services"]:
        if s["kind"] == kind and (not address or s["address"] == address):
            pid = int(s.get("pid", 0))
            if pid > 0 and pid != os.getpid() and _pid_alive(pid):
                os.kill(pid, signal.SIGTERM)
            n += 1
        else:
            keep.append(s)
    st["services"] = keep
    save_state(st)
    print(f"stopped {n} {kind} service(s)")
    return 0 if n else 1


def cmd_logs(name: str, lines: int) -> int:
    for s in load_state()["services"]:
        if name in (s["address"], s["kind"], s.get("name")) and s.get("log"):
            try:
                with open(s["log"]) as f:
                    print("".join(f.readlines()[-lines:]), end="")
                return 0
            except OSError as e:
                print(f"cannot read {s['log']}: {e}")
                return 1
    print(f"no recorded service '{name}' with a log file")
    return 1


def _serve_forever(stop) -> None:
    try:
        threading.Event().wait()
    except KeyboardInterrupt:
        pass
    stop()


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="areal_b200.v2.cli")
    sub = ap.add_subparsers(dest="service", required=True)
    inf = sub.add_parser("inference")
    inf.add_argument("action", choices=["serve", "status", "ps", "models", "stop"])
    inf.add_argument("--address", default="")
    inf.add_argument("--model-path", default="")
    inf.add_argument("--preset", default="")
    inf.add_argument("--port", type=int, default=0)
    inf.add_argument("--host", default="127.0.0.1")
    wu = sub.add_parser("weight-update")
    wu.add_argument("action", choices=["serve", "status"])
    wu.add_argument("--port", type=int, default=0)
    wu.add_argument("--host", default="127.0.0.1")
    dat = sub.add_parser("data")
    dat.add_argument("action", choices=["serve", "status", "ps", "stop"])
    dat.add_argument("role", nargs="?", default="worker", choices=["worker", "router", "gateway"])
    dat.add_argument("--router", default=None)
    dat.add_argument("--admin-key", default=None)
    dat.add_argument("--port", type=int, default=0)
    dat.add_argument("--host", default="127.0.0.1")
    dat.add_argument("--address", default="")
    sbx = sub.add_parser("sandbox")
    sbx.add_argument("action", choices=["serve", "status", "ps", "stop"])
    sbx.add_argument("--api-key", default=None)
    sbx.add_argument("--port", type=int, default=0)
    sbx.add_argument("--host", default="127.0.0.1")
    sbx.add_argument("--address", default="")
    trn = sub.add_parser("training")
    trn.add_argument("action", choices=["run"])
    trn.add_argument("script")
    trn.add_argument("rest", nargs=argparse.REMAINDER)
    lg = sub.add_parser("logs")
    lg.add_argument("name")
    lg.add_argument("-n", "--lines", type=int, default=50)
    stp = sub.add_parser("state")
    stp.add_argument("action", choices=["show", "clear"])
    a = ap.parse_args(argv)
    if a.service == "logs":
        return cmd_logs(a.name, a.lines)
    if a.service == "training":
        from ..infra.launcher import local as launcher

        return int(launcher.main([a.script] + list(a.rest)) or 0)
    if a.service in ("inference", "data", "sandbox") and a.action == "ps":
        return cmd_ps(a.service)
    if a.service in ("inference", "data", "sandbox") and a.action == "stop":
        return cmd_stop(a.service, a.address)
    if a.service == "inference" and a.action == "models":
        rc = 1
        for s_ in load_state()["services"]:
            if s_["kind"] == "inference" and (not a.address or s_["address"] == a.address):
                try:
                    print(s_["address"], json.dumps(call(f"http://{s_['address']}/v1/models", timeout=5)))
                    rc = 0
                except HTTPError as e:
                    print(s_["address"], "DOWN", e.message[:80])
        return rc
    if a.service == "data" and a.action == "serve":
        from ..infra.data_service.service import DataGateway, DataRouter, DataWorker

        if a.role == "worker":
            svc = DataWorker(a.host, a.port or None, a.admin_key).start()
            if a.router:
                call(f"http://{a.router}/register", {"address": svc.address}, api_key=a.admin_key, retries=5)
        elif a.role == "router":
            svc = DataRouter(a.host, a.port or None, a.admin_key, poll_interval_s=5.0).start()
        else:
            if not a.router:
                ap.error("data serve gateway needs --router")
            svc = DataGateway(a.router, a.host, a.port or None, a.admin_key).start()
        record("data", svc.address, role=a.role)
        print(f"DATA_{a.role.upper()}_READY {svc.address}", flush=True)
        _serve_forever(svc.stop)
        return 0
    if a.service == "sandbox" and a.action == "serve":
        from ..infra.sandbox import SandboxServer

        svc = SandboxServer(host=a.host, port=a.port or None, api_key=a.api_key).start()
        record("sandbox", svc.address)
        print(f"SANDBOX_READY {svc.address}", flush=True)
        _serve_forever(svc.stop)
        return 0
    if a.service in ("data", "sandbox"):
        return cmd_status(a.service)
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
