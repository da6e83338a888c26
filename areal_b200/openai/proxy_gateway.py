"""One address in front of several OpenAI-compatible proxies.

Agents outside the training job talk to ONE url. ``POST /rl/start_session`` (admin key) opens a
session on the backend proxy with the fewest open sessions and returns its key; every later
request that carries the key (chat completions, messages, responses, rewards, end of session) is
relayed to the backend that owns it, streamed replies included; ``/rl/export_trajectories`` is
relayed to the owner and closes the mapping. Reference: the gateway that
``RolloutController.start_proxy_gateway`` puts in front of its proxy workers
(``areal/infra/controller/rollout_controller.py:496-577``,
``areal/experimental/openai/proxy/proxy_gateway.py``).
"""
from __future__ import annotations

import json
import threading
import urllib.error
import urllib.request
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer
from typing import Optional

from ..utils import logging as alog
from ..utils.network import find_free_ports

logger = alog.getLogger("proxy_gateway")


class ProxyGateway:
    def __init__(self, proxy_addrs: list[str], admin_api_key: Optional[str] = None, host: str = "127.0.0.1", port: Optional[int] = None,
                 timeout_s: float = 3600.0):
        if not proxy_addrs:
            raise ValueError("the gateway needs at least one backend proxy")
        self.backends = [a.rstrip("/") if a.startswith("http") else f"http://{a}" for a in proxy_addrs]
        self.backends = [b[:-3] if b.endswith("/v1") else b for b in self.backends]
        self.admin_api_key = admin_api_key
        self.host, self.port = host, port or find_free_ports(1)[0]
        self.timeout_s = timeout_s
        self._owner: dict[str, int] = {}
        self._open = [0] * len(self.backends)
        self._lock = threading.Lock()
        self._srv: Optional[ThreadingHTTPServer] = None

    @property
    def addr(self) -> str:
        return f"http://{self.host}:{self.port}"

    @property
    def base_url(self) -> str:
        return self.addr + "/v1"

    # ---- routing state
    def _pick(self) -> int:
        with self._lock:
            i = min(range(len(self.backends)), key=lambda j: (self._open[j], j))
            self._open[i] += 1
            return i

    def _bind(self, key: str, i: int) -> None:
        with self._lock:
            self._owner[key] = i

    def _unbind(self, key: str) -> None:
        with self._lock:
            i = self._owner.pop(key, None)
            if i is not None:
                self._open[i] = max(0, self._open[i] - 1)

    def _owner_of(self, key: Optional[str]) -> int:
        with self._lock:
            i = self._owner.get(key or "")
        if i is None:
            raise PermissionError("unknown session key")
        return i

    def sessions(self) -> list[int]:
        with self._lock:
            return list(self._open)

    # ---- relay
    def _forward(self, i: int, method: str, path: str, body: bytes, headers: dict):
        """Returns (status, content type, payload bytes) of the backend's reply."""
        req = urllib.request.Request(self.backends[i] + path, data=body if method != "GET" else None, method=method,
                                     headers={k: v for k, v in headers.items() if v is not None})
        try:
            with urllib.request.urlopen(req, timeout=self.timeout_s) as r:
                return r.status, r.headers.get("Content-Type", "application/json"), r.read()
        except urllib.error.HTTPError as e:
            return e.code, e.headers.get("Content-Type", "application/json"), e.read()

    def start(self):
        gw = self

        class H(BaseHTTPRequestHandler):
            protocol_version = "HTTP/1.1"

            def log_message(self, *a):
                pass

            def _key(self) -> Optional[str]:
                a = self.headers.get("Authorization", "")
                if a.lower().startswith("bearer "):
                    return a[7:].strip()
                return self.headers.get("x-api-key")

            def _send(self, code: int, ctype: str, payload: bytes):
                self.send_response(code)
                self.send_header("Content-Type", ctype)
                self.send_header("Content-Length", str(len(payload)))
                self.end_headers()
                self.wfile.write(payload)

            def _json(self, code: int, obj):
                self._send(code, "application/json", json.dumps(obj).encode())

            def do_GET(self):
                if self.path in ("/health", "/v1/health"):
                    return self._json(200, {"status": "ok", "backends": gw.backends, "open_sessions": gw.sessions()})
                if self.path in ("/v1/models", "/models"):
                    return self._send(*gw._forward(0, "GET", self.path, b"", {}))
                self._json(404, {"error": "unknown route"})

            def do_POST(self):
                n = int(self.headers.get("Content-Length", "0"))
                raw = self.rfile.read(n) if n else b""
                path = self.path.split("?")[0].rstrip("/")
                hdr = {"Content-Type": "application/json", "Authorization": self.headers.get("Authorization"),
                       "x-api-key": self.headers.get("x-api-key")}
                try:
                    if path == "/rl/start_session":
                        if gw.admin_api_key and self._key() != gw.admin_api_key:
                            raise PermissionError("admin key required")
                        i = gw._pick()
                        code, ctype, payload = gw._forward(i, "POST", path, raw, hdr)
                        if code == 200:
                            key = json.loads(payload)["api_key"]
                            gw._bind(key, i)
                            payload = json.dumps({"api_key": key, "base_url": gw.base_url}).encode()
                        else:
                            with gw._lock:
                                gw._open[i] = max(0, gw._open[i] - 1)
                        return self._send(code, ctype, payload)
                    if path == "/rl/export_trajectories":
                        body = json.loads(raw) if raw else {}
                        key = body.get("api_key") or self._key()
                        i = gw._owner_of(key)
                        out = gw._forward(i, "POST", path, raw, hdr)
                        if out[0] == 200:
                            gw._unbind(key)
                        return self._send(*out)
                    i = gw._owner_of(self._key())
                    return self._send(*gw._forward(i, "POST", path, raw, hdr))
                except PermissionError as e:
                    self._json(401, {"error": str(e)})
                except (urllib.error.URLError, ConnectionError, OSError) as e:
                    self._json(502, {"error": f"backend unreachable: {e!r}"})

        self._srv = ThreadingHTTPServer((self.host, self.port), H)
        self._srv.daemon_threads = True
        threading.Thread(target=self._srv.serve_forever, daemon=True, name="proxy-gateway").start()
        logger.info("proxy gateway on %s over %d backends", self.addr, len(self.backends))
        return self

    def stop(self):
        if self._srv is not None:
            self._srv.shutdown()
            self._srv.server_close()
            self._srv = None
