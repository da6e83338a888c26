"""Session-affine router: new sessions go to the least-loaded healthy data proxy; every later
request of a session goes to the proxy that owns it. Reference:
``areal/v2/inference_service/router/app.py``."""
from __future__ import annotations

import threading
from typing import Optional

from ..common import HTTPError, JsonService, call


class Router:
    def __init__(self, host: str = "127.0.0.1", port: Optional[int] = None, policy: str = "least_sessions"):
        self.workers: dict[str, dict] = {}         # address -> {"sessions": int, "healthy": bool}
        self.session_to_worker: dict[str, str] = {}
        self.policy = policy
        self._rr = 0
        self._lock = threading.Lock()
        self.svc = JsonService("router", host, port)
        self._install()

    def pick(self) -> str:
        with self._lock:
            live = [a for a, w in self.workers.items() if w["healthy"]]
            if not live:
                raise HTTPError(503, "no healthy inference worker registered")
            if self.policy == "round_robin":
                a = live[self._rr % len(live)]
                self._rr += 1
            else:
                a = min(live, key=lambda x: (self.workers[x]["sessions"], x))
            self.workers[a]["sessions"] += 1
            return a

    def owner(self, session_id: Optional[str]) -> str:
        with self._lock:
            a = self.session_to_worker.get(session_id or "")
        if a is None:
            raise HTTPError(404, "unknown session")
        return a

    def _install(self):
        svc = self.svc

        @svc.route("GET", "/health")
        def health(body, ctx):
            return {"status": "ok", "workers": self.workers, "sessions": len(self.session_to_worker)}

        @svc.route("POST", "/register")
        def register(body, ctx):
            with self._lock:
                self.workers.setdefault(body["address"], {"sessions": 0, "healthy": True})["healthy"] = True
            return {"ok": True, "workers": len(self.workers)}

        @svc.route("POST", "/unregister")
        def unregister(body, ctx):
            with self._lock:
                self.workers.pop(body["address"], None)
                for k in [k for k, v in self.session_to_worker.items() if v == body["address"]]:
                    del self.session_to_worker[k]
            return {"ok": True}

        @svc.route("POST", "/route/new_session")
        def new_session(body, ctx):
            a = self.pick()
            return {"address": a}

        @svc.route("POST", "/route/bind")
        def bind(body, ctx):
            with self._lock:
                self.session_to_worker[body["session_id"]] = body["address"]
            return {"ok": True}

        @svc.route("POST", "/route/lookup")
        def lookup(body, ctx):
            return {"address": self.owner(body.get("session_id"))}

        @svc.route("POST", "/route/release")
        def release(body, ctx):
            with self._lock:
                a = self.session_to_worker.pop(body.get("session_id"), None)
                if a in self.workers:
                    self.workers[a]["sessions"] = max(0, self.workers[a]["sessions"] - 1)
            return {"ok": True}

        @svc.route("POST", "/health_check")
        def health_check(body, ctx):
            for a in list(self.workers):
                try:
                    ok = call(f"http://{a}/health", timeout=3).get("status") == "ok"
                except HTTPError:
                    ok = False
                with self._lock:
                    if a in self.workers:
                        self.workers[a]["healthy"] = ok
            return {"workers": self.workers}

    def start(self):
        self.svc.start()
        return self

    def stop(self):
        self.svc.stop()

    @property
    def address(self) -> str:
        return self.svc.address
