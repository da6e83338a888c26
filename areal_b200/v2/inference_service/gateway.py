"""Public entry of the inference service: OpenAI-compatible chat completions plus the RL
session routes, in front of a router and any number of data proxies. The gateway is
stateless: session ownership lives in the router. Reference:
``areal/v2/inference_service/gateway/app.py``."""
from __future__ import annotations

from typing import Optional

from ..common import HTTPError, JsonService, call


class Gateway:
    def __init__(self, router_address: str, admin_key: str = "areal-admin-key", host: str = "127.0.0.1", port: Optional[int] = None):
        self.router, self.admin_key = router_address, admin_key
        self.svc = JsonService("gateway", host, port)
        self._install()

    def _admin(self, ctx):
        if ctx.api_key != self.admin_key:
            raise HTTPError(401, "admin key required")

    def _workers(self) -> list[str]:
        return [a for a, w in call(f"http://{self.router}/health")["workers"].items() if w["healthy"]]

    def _fan(self, path: str, body: dict) -> dict:
        res = {}
        for a in self._workers():
            res[a] = call(f"http://{a}{path}", body)
        return res

    def _install(self):
        svc = self.svc

        @svc.route("GET", "/health")
        def health(body, ctx):
            return {"status": "ok", "router": call(f"http://{self.router}/health")}

        @svc.route("POST", "/rl/start_session")
        def start(body, ctx):
            self._admin(ctx)
            a = call(f"http://{self.router}/route/new_session", {})["address"]
            s = call(f"http://{a}/rl/start_session", body)
            call(f"http://{self.router}/route/bind", {"session_id": s["session_id"], "address": a})
            return {**s, "base_url": f"{self.svc.url}/v1"}

        def forward(path):
            def fn(body, ctx):
                a = call(f"http://{self.router}/route/lookup", {"session_id": ctx.api_key})["address"]
                if body.get("stream"):
                    # relay the worker's event stream as it arrives (reference: areal/v2/inference_service/gateway/streaming.py)
                    from ..common import SSE, sse_lines

                    return SSE(sse_lines(f"http://{a}{path}", body, api_key=ctx.api_key))
                return call(f"http://{a}{path}", body, api_key=ctx.api_key)
            return fn
        svc.route("POST", "/v1/chat/completions")(forward("/chat/completions"))
        svc.route("POST", "/chat/completions")(forward("/chat/completions"))
        svc.route("POST", "/rl/set_reward")(forward("/rl/set_reward"))
        svc.route("POST", "/v1/messages")(forward("/v1/messages"))
        svc.route("POST", "/v1/responses")(forward("/v1/responses"))

        def any_worker(path):
            def fn(body, ctx):
                ws = self._workers()
                if not ws:
                    raise HTTPError(503, "no inference worker registered")
                return call(f"http://{ws[0]}{path}", body)
            return fn
        svc.route("POST", "/tokenize")(any_worker("/tokenize"))
        svc.route("POST", "/detokenize")(any_worker("/detokenize"))

        @svc.route("POST", "/rl/end_session")
        def end(body, ctx):
            a = call(f"http://{self.router}/route/lookup", {"session_id": ctx.api_key})["address"]
            r = call(f"http://{a}/rl/end_session", body, api_key=ctx.api_key)
            call(f"http://{self.router}/route/release", {"session_id": ctx.api_key})
            return r

        @svc.route("POST", "/export_trajectories")
        def export(body, ctx):
            self._admin(ctx)
            sessions = []
            for a in self._workers():
                sessions += call(f"http://{a}/export_trajectories", body)["sessions"]
            return {"sessions": sessions}

        for name in ("pause_generation", "continue_generation", "set_version", "release_memory", "resume_memory"):
            def ctl(body, ctx, name=name):
                self._admin(ctx)
                return {"workers": self._fan(f"/{name}", body)}
            svc.route("POST", f"/{name}")(ctl)

    def start(self):
        self.svc.start()
        return self

    def stop(self):
        self.svc.stop()

    @property
    def address(self) -> str:
        return self.svc.address
