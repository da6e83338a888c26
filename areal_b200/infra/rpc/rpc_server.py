"""Worker-side RPC server: hosts engines created on request and executes their methods.

``python -m areal_b200.infra.rpc.rpc_server --port P [--host H] [--role R --index I]``

Routes (JSON bodies in the envelope of :mod:`serialization`):

    GET  /health                      liveness + hosted engines
    POST /configure  {env, seed}      process-level settings
    POST /set_env    {env}            environment variables (RANK, MASTER_ADDR, ...)
    POST /alloc_ports {count}         free ports on this host (never handed out twice by one server)
    POST /fork {role, worker_index, raw_cmd, env}   start a sibling process on this node (one per role/index)
    POST /kill_forked_worker {role, worker_index}   end it (its whole process group)
    GET  /forked                      the children this server started, with their state
    POST /data/batch {shard_ids}      several shards in one reply
    POST /create_engine {name, cls, args, kwargs}
    POST /call {name, method, args, kwargs, return_rtensor, direct}   run ``engine.method`` in the engine thread
    PUT  /data/<shard_id>  (torch.save bytes)   GET /data/<shard_id>   POST /data/clear {shard_ids}
    POST /kill                        exit the process (children started by /fork are ended first)

The fork / kill / port routes are the node-guard role of the reference
(``areal/infra/rpc/guard/app.py:193-416``): a controller that colocates a second role with a
worker (a reference model beside the actor, a proxy beside a rollout server) asks the worker's
server to start it, so that it lands on the same node and shares its GPU visibility.

All engine calls are executed by ONE engine thread in arrival order, which serialises
collectives exactly like the reference's guard (``areal/infra/rpc/guard/engine_blueprint.py:115-181``).
Arguments of type :class:`RTensor` are materialised before the call; a dict-of-tensors result
is kept in the local shard store and returned as an :class:`RTensor` when the caller asks for
it (``return_rtensor``).
"""
from __future__ import annotations

import argparse
import json
import os
import queue
import signal
import subprocess
import sys
import tempfile
import threading
import traceback
from concurrent.futures import Future
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer
from typing import Any

import torch

from ...utils import logging as alog
from ...utils.dynamic_import import import_from_string
from ...utils.network import find_free_ports, gethostip
from . import rtensor as RT
from .hosted import HOSTED_ENGINES
from .serialization import deserialize_value, serialize_value

logger = alog.getLogger("rpc_server")


class EngineHost:
    def __init__(self, addr: str):
        self.addr = addr
        self.engines: dict[str, Any] = {}
        self._q: "queue.Queue[tuple]" = queue.Queue()
        self._thread = threading.Thread(target=self._loop, name="engine-thread", daemon=True)
        self._thread.start()

    def _loop(self):
        while True:
            fn, fut = self._q.get()
            if fn is None:
                return
            try:
                fut.set_result(fn())
            except BaseException as e:  # returned to the caller
                fut.set_exception(e)

    def run(self, fn, timeout=None):
        fut: Future = Future()
        self._q.put((fn, fut))
        return fut.result(timeout=timeout)

    def create_engine(self, name: str, cls_path: str, args, kwargs):
        def make():
            cls = import_from_string(cls_path)
            self.engines[name] = cls(*args, **kwargs)
            HOSTED_ENGINES[name] = self.engines[name]
            return True
        return self.run(make)

    def call(self, name: str, method: str, args, kwargs, return_rtensor: bool = False, direct: bool = False):
        def materialise(x):
            if isinstance(x, RT.RTensor):
                return RT.fetch(x, my_addr=self.addr)
            if isinstance(x, dict):
                return {k: materialise(v) for k, v in x.items()}
            if isinstance(x, (list, tuple)):
                return type(x)(materialise(v) for v in x)
            return x

        def do():
            eng = self.engines[name]
            target = eng
            for part in method.split("."):
                target = getattr(target, part)
            res = target(*materialise(args), **materialise(kwargs)) if callable(target) else target
            if isinstance(res, Future):
                res = res.result()
            if res is eng:  # fluent ``return self``
                return None
            if return_rtensor and isinstance(res, dict) and res and all(isinstance(v, torch.Tensor) or not isinstance(v, dict)
                                                                        for v in res.values()):
                return RT.remotize(res, self.addr)
            return res
        # ``direct`` calls run in the HTTP handler thread: for thread-safe, possibly blocking
        # methods (submit / wait_for_task of an inference engine) that must not queue behind
        # one another in the engine thread
        return do() if direct else self.run(do)


class ForkedWorkers:
    """Children started on behalf of a controller, keyed by (role, index)."""

    def __init__(self, log_dir: str | None = None):
        self._procs: dict[tuple[str, int], subprocess.Popen] = {}
        self._lock = threading.Lock()
        self.log_dir = log_dir or os.path.join(tempfile.gettempdir(), f"areal_forked_{os.getpid()}")
        self.ports: set[int] = set()

    def alloc_ports(self, count: int) -> list[int]:
        if not isinstance(count, int) or count <= 0:
            raise ValueError("'count' must be a positive integer")
        with self._lock:
            got = find_free_ports(count, exclude=self.ports)
            self.ports.update(got)
        return got

    def fork(self, role: str, index: int, raw_cmd: list, env: dict | None = None) -> int:
        if not role or not isinstance(raw_cmd, list) or not raw_cmd:
            raise ValueError("'role' and a non-empty 'raw_cmd' list are required")
        key = (str(role), int(index))
        with self._lock:
            old = self._procs.get(key)
            if old is not None and old.poll() is None:
                raise ValueError(f"worker {role}/{index} is already running (pid {old.pid})")
            os.makedirs(self.log_dir, exist_ok=True)
            log = open(os.path.join(self.log_dir, f"{role}_{index}.log"), "ab")
            child_env = dict(os.environ)
            child_env.update({str(k): str(v) for k, v in (env or {}).items()})
            # its own session: ending the child ends what the child started, and nothing else
            p = subprocess.Popen([str(c) for c in raw_cmd], env=child_env, stdout=log, stderr=subprocess.STDOUT,
                                 stdin=subprocess.DEVNULL, start_new_session=True)
            log.close()
            self._procs[key] = p
        logger.info("forked %s/%d as pid %d: %s", role, index, p.pid, " ".join(map(str, raw_cmd)))
        return p.pid

    @staticmethod
    def _end(p: subprocess.Popen, grace_s: float = 5.0) -> None:
        if p.poll() is not None:
            return
        for sig in (signal.SIGTERM, signal.SIGKILL):
            try:
                os.killpg(p.pid, sig)         # the child leads its own process group (start_new_session)
            except ProcessLookupError:
                return
            try:
                p.wait(timeout=grace_s)
                return
            except subprocess.TimeoutExpired:
                continue

    def kill(self, role: str, index: int) -> bool:
        with self._lock:
            p = self._procs.pop((str(role), int(index)), None)
        if p is None:
            return False
        self._end(p)
        return True

    def kill_all(self) -> None:
        with self._lock:
            procs, self._procs = list(self._procs.values()), {}
        for p in procs:
            self._end(p)

    def status(self) -> list[dict]:
        with self._lock:
            return [{"role": r, "worker_index": i, "pid": p.pid, "returncode": p.poll()} for (r, i), p in sorted(self._procs.items())]


def make_handler(host: EngineHost, stop_event: threading.Event, forked: "ForkedWorkers | None" = None):
    forked = forked or ForkedWorkers()

    class Handler(BaseHTTPRequestHandler):
        protocol_version = "HTTP/1.1"

        def log_message(self, *a):  # quiet
            pass

        def _send(self, code: int, body: bytes, ctype="application/json"):
            self.send_response(code)
            self.send_header("Content-Type", ctype)
            self.send_header("Content-Length", str(len(body)))
            self.end_headers()
            self.wfile.write(body)

        def _json(self, code: int, obj):
            self._send(code, json.dumps(obj).encode())

        def _body(self) -> bytes:
            n = int(self.headers.get("Content-Length", "0"))
            return self.rfile.read(n) if n else b""

        def do_GET(self):
            if self.path == "/health":
                return self._json(200, {"status": "ok", "engines": sorted(host.engines), "pid": os.getpid(), "shards": len(RT.LOCAL_STORE)})
            if self.path == "/forked":
                return self._json(200, {"workers": forked.status()})
            if self.path.startswith("/data/"):
                sid = self.path[len("/data/"):]
                try:
                    return self._send(200, RT.dumps_batch(RT.LOCAL_STORE.get(sid)), "application/octet-stream")
                except KeyError:
                    return self._json(404, {"error": f"shard {sid} not found"})
            self._json(404, {"error": "unknown route"})

        def do_PUT(self):
            if self.path.startswith("/data/"):
                sid = self.path[len("/data/"):]
                RT.LOCAL_STORE.put(RT.loads_batch(self._body()), sid)
                return self._json(200, {"shard_id": sid})
            self._json(404, {"error": "unknown route"})

        def do_POST(self):
            try:
                raw = self._body()
                req = deserialize_value(json.loads(raw)) if raw else {}
                if self.path == "/configure" or self.path == "/set_env":
                    for k, v in (req.get("env") or {}).items():
                        os.environ[str(k)] = str(v)
                    if req.get("seed") is not None:
                        from ...utils.seeding import set_random_seed

                        set_random_seed(int(req["seed"]), req.get("seed_key", ""))
                    return self._json(200, {"ok": True})
                if self.path == "/alloc_ports":
                    try:
                        return self._json(200, {"status": "success", "ports": forked.alloc_ports(req.get("count", 1)), "host": gethostip()})
                    except ValueError as e:
                        return self._json(400, {"error": str(e)})
                if self.path == "/fork":
                    try:
                        pid = forked.fork(req.get("role"), req.get("worker_index", 0), req.get("raw_cmd"), req.get("env"))
                    except ValueError as e:
                        return self._json(400, {"error": str(e)})
                    return self._json(200, {"status": "success", "host": gethostip(), "pid": pid})
                if self.path == "/kill_forked_worker":
                    if req.get("role") is None:
                        return self._json(400, {"error": "Missing 'role' field in request"})
                    if not forked.kill(req["role"], req.get("worker_index", 0)):
                        return self._json(404, {"error": f"no forked worker {req['role']}/{req.get('worker_index', 0)}"})
                    return self._json(200, {"status": "success"})
                if self.path == "/data/batch":
                    out, missing = {}, []
                    for sid in req.get("shard_ids", []):
                        try:
                            out[sid] = RT.LOCAL_STORE.get(sid)
                        except KeyError:
                            missing.append(sid)
                    if missing:
                        return self._json(404, {"error": "shards not found", "missing": missing})
                    return self._send(200, RT.dumps_batch(out), "application/octet-stream")
                if self.path == "/create_engine":
                    host.create_engine(req["name"], req["cls"], req.get("args", []), req.get("kwargs", {}))
                    return self._json(200, {"ok": True})
                if self.path == "/call":
                    res = host.call(req["name"], req["method"], req.get("args", []), req.get("kwargs", {}),
                                    bool(req.get("return_rtensor", False)), bool(req.get("direct", False)))
                    return self._json(200, {"result": serialize_value(res)})
                if self.path == "/data/clear":
                    ids = req.get("shard_ids")
                    if ids is None:
                        RT.LOCAL_STORE.clear()
                        return self._json(200, {"deleted": "all"})
                    return self._json(200, {"deleted": RT.LOCAL_STORE.delete(ids)})
                if self.path == "/kill":
                    forked.kill_all()
                    self._json(200, {"ok": True})
                    stop_event.set()
                    return
                self._json(404, {"error": "unknown route"})
            except BaseException as e:
                self._json(500, {"error": repr(e), "traceback": traceback.format_exc()})

    return Handler


def serve(host_ip: str, port: int) -> None:
    addr = f"{host_ip}:{port}"
    eh = EngineHost(addr)
    stop = threading.Event()
    srv = ThreadingHTTPServer((host_ip if host_ip != gethostip() else "0.0.0.0", port), make_handler(eh, stop))
    srv.daemon_threads = True
    t = threading.Thread(target=srv.serve_forever, daemon=True)
    t.start()
    logger.info("rpc worker listening on %s (pid %d)", addr, os.getpid())
    stop.wait()
    for e in eh.engines.values():
        try:
            e.destroy()
        except Exception:
            pass
    srv.shutdown()


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--port", type=int, required=True)
    ap.add_argument("--role", default="worker")
    ap.add_argument("--index", type=int, default=0)
    ap.add_argument("--announce", default="", help="name_resolve key prefix under which '<prefix>/<index>' -> host:port is published")
    a = ap.parse_args(argv)
    if a.port == 0:
        a.port = find_free_ports(1)[0]
    if a.announce:
        from ...utils import name_resolve

        name_resolve.add(f"{a.announce}/{a.index}", f"{a.host}:{a.port}", replace=True)
    serve(a.host, a.port)
    os._exit(0)


if __name__ == "__main__":
    main()
