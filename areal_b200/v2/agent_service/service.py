from __future__ import annotations

import threading
import time
import uuid
from dataclasses import dataclass, field
from typing import Any, Callable, Optional

from ...utils import logging as alog
from ...utils.dynamic_import import import_from_string
from ..common import HTTPError, JsonService, call

logger = alog.getLogger("agent_service")


@dataclass
class SessionInfo:
    """What an agent gets besides the message: where the model lives and which key records its calls."""
    session_key: str
    base_url: str = ""                  # OpenAI-compatible endpoint of the inference gateway
    api_key: str = ""                   # per-session key issued by ``/rl/start_session``
    history: list = field(default_factory=list)
    metadata: dict = field(default_factory=dict)


class AgentWorker:
    """Hosts one agent callable. ``POST /turn {session_key, message, base_url, api_key, history}``."""

    def __init__(self, agent: Any, host: str = "127.0.0.1", port: Optional[int] = None):
        self.agent: Callable = import_from_string(agent) if isinstance(agent, str) else agent
        self.svc = JsonService("agent-worker", host, port)
        self.turns = 0

        @self.svc.route("GET", "/health")
        def health(body, ctx):
            return {"status": "ok", "turns": self.turns}

        @self.svc.route("POST", "/turn")
        def turn(body, ctx):
            s = SessionInfo(session_key=body["session_key"], base_url=body.get("base_url", ""), api_key=body.get("api_key", ""),
                            history=list(body.get("history") or []), metadata=dict(body.get("metadata") or {}))
            out = self.agent(body["message"], s)
            self.turns += 1
            return out if isinstance(out, dict) else {"text": str(out)}

    def start(self):
        self.svc.start()
        return self

    def stop(self):
        self.svc.stop()

    @property
    def address(self) -> str:
        return self.svc.address


class AgentGateway:
    def __init__(self, workers: list[str], inference_gateway: str = "", admin_key: str = "areal-admin-key", host: str = "127.0.0.1",
                 port: Optional[int] = None, turn_timeout: float = 600.0):
        self.workers, self.inference, self.admin_key, self.turn_timeout = list(workers), inference_gateway, admin_key, turn_timeout
        self.svc = JsonService("agent-gateway", host, port)
        self._lock = threading.Lock()
        self._sessions: dict[str, dict] = {}
        self._runs: dict[str, dict] = {}
        self._rr = 0
        self._install()

    # ---- session bookkeeping
    def _session(self, key: str) -> dict:
        with self._lock:
            s = self._sessions.get(key)
            if s is None:
                api_key = ""
                if self.inference:
                    api_key = call(f"http://{self.inference}/rl/start_session", {"task_id": key}, api_key=self.admin_key)["api_key"]
                w = self.workers[self._rr % len(self.workers)]      # a session stays on one worker
                self._rr += 1
                s = self._sessions[key] = dict(key=key, worker=w, api_key=api_key, history=[], queue=[], active=None, ended=False)
            return s

    def _start_run(self, s: dict, message: str, mode: str) -> dict:
        run = dict(run_id=uuid.uuid4().hex, session_key=s["key"], status="running", message=message, result=None, error=None,
                   queue_mode=mode, created=time.time())
        self._runs[run["run_id"]] = run
        s["active"] = run["run_id"]
        threading.Thread(target=self._execute, args=(s, run), daemon=True, name=f"agent-run-{run['run_id'][:6]}").start()
        return run

    def _execute(self, s: dict, run: dict):
        try:
            base = f"http://{self.inference}/v1" if self.inference else ""
            res = call(f"http://{s['worker']}/turn", dict(session_key=s["key"], message=run["message"], base_url=base, api_key=s["api_key"],
                                                          history=s["history"]), timeout=self.turn_timeout)
            run["result"], run["status"] = res, "ok"
            s["history"] += [{"role": "user", "content": run["message"]}, {"role": "assistant", "content": res.get("text", "")}]
        except Exception as e:  # the run fails, the session stays usable
            run["error"], run["status"] = repr(e), "error"
        nxt = None
        with self._lock:
            s["active"] = None
            if s["queue"] and not s["ended"]:
                mode = s["queue"][0][1]
                if mode == "collect":                       # everything that piled up becomes one follow-up turn
                    msgs = [m for m, _ in s["queue"]]
                    s["queue"].clear()
                    nxt = ("\n".join(msgs), mode)
                else:
                    nxt = s["queue"].pop(0)
                follow = self._start_run(s, nxt[0], nxt[1])
                run["followup_run_id"] = follow["run_id"]

    # ---- routes
    def _install(self):
        svc = self.svc

        @svc.route("GET", "/health")
        def health(body, ctx):
            return {"status": "ok", "workers": self.workers, "sessions": len(self._sessions)}

        @svc.route("POST", "/agent/run")
        def run(body, ctx):
            key, msg = body.get("session_key") or uuid.uuid4().hex, body["message"]
            mode = body.get("queue_mode", "collect")
            if mode not in ("collect", "followup"):
                raise HTTPError(400, f"unknown queue_mode '{mode}'")
            s = self._session(key)
            if s["ended"]:
                raise HTTPError(409, "session has ended")
            with self._lock:
                if s["active"] is not None:
                    s["queue"].append((msg, mode))
                    return {"session_key": key, "status": "queued", "active_run_id": s["active"], "queued": len(s["queue"])}
                r = self._start_run(s, msg, mode)
            return {"session_key": key, "run_id": r["run_id"], "status": "running"}

        @svc.route("GET", "/agent/runs/{run_id}")
        def get_run(body, ctx):
            r = self._runs.get(ctx.params["run_id"])
            if r is None:
                raise HTTPError(404, "unknown run")
            return {k: r.get(k) for k in ("run_id", "session_key", "status", "result", "error", "followup_run_id", "queue_mode")}

        @svc.route("POST", "/agent/sessions/{key}/end")
        def end(body, ctx):
            s = self._sessions.get(ctx.params["key"])
            if s is None:
                raise HTTPError(404, "unknown session")
            s["ended"] = True
            out = {"session_key": s["key"], "turns": len(s["history"]) // 2}
            if self.inference and s["api_key"]:
                if "reward" in body:
                    call(f"http://{self.inference}/rl/set_reward", {"reward": float(body["reward"])}, api_key=s["api_key"])
                out["inference"] = call(f"http://{self.inference}/rl/end_session", {}, api_key=s["api_key"])
            return out

    def wait_run(self, run_id: str, timeout: float = 60.0) -> dict:
        t0 = time.time()
        while time.time() - t0 < timeout:
            r = self._runs[run_id]
            if r["status"] != "running":
                return r
            time.sleep(0.01)
        raise TimeoutError(run_id)

    def start(self):
        self.svc.start()
        return self

    def stop(self):
        self.svc.stop()

    @property
    def address(self) -> str:
        return self.svc.address


class AgentController:
    """Starts ``n_workers`` agent workers and one gateway in this process; ``close`` stops them."""

    def __init__(self, agent: Any, n_workers: int = 1, inference_gateway: str = "", admin_key: str = "areal-admin-key"):
        self.workers = [AgentWorker(agent).start() for _ in range(n_workers)]
        self.gateway = AgentGateway([w.address for w in self.workers], inference_gateway, admin_key).start()

    def run(self, session_key: str, message: str, queue_mode: str = "collect", wait: bool = True, timeout: float = 60.0) -> dict:
        r = call(f"http://{self.gateway.address}/agent/run", dict(session_key=session_key, message=message, queue_mode=queue_mode))
        if wait and "run_id" in r:
            return self.gateway.wait_run(r["run_id"], timeout)
        return r

    def close(self):
        self.gateway.stop()
        for w in self.workers:
            w.stop()
