"""Minimal JSON-over-HTTP service scaffold shared by the v2 services (stdlib only): a route
table of ``(method, path) -> handler(body, ctx) -> (status, json)`` served by a threading HTTP
server, bearer-key extraction, and a small JSON client with retries.

The reference builds its services on FastAPI / Flask (``areal/v2/*/app.py``); the routes and
payloads here follow those files, the web framework does not matter to callers."""
from __future__ import annotations

import json
import threading
import time
import urllib.error
import urllib.request
from dataclasses import dataclass
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer
from typing import Any, Callable, Optional

from ..utils import logging as alog
from ..utils.network import find_free_ports

logger = alog.getLogger("v2")


class HTTPError(Exception):
    def __init__(self, status: int, message: str):
        super().__init__(message)
        self.status, self.message = status, message


@dataclass
class RequestCtx:
    api_key: Optional[str]
    path: str
    params: dict[str, str]
    headers: Any


class SSE:
    """A handler's answer that is streamed as server-sent events over chunked transfer encoding. ``events``
    yields payload dicts, raw strings (sent as they are, e.g. ``[DONE]``) or ``(event name, payload)`` pairs."""

    def __init__(self, events):
        self.events = events


def sse_lines(url: str, body: dict, api_key: Optional[str] = None, timeout: float = 600.0):
    """POSTs ``body`` and yields the events of the streamed answer as ``(event name or None, data string)``."""
    headers = {"Content-Type": "application/json", "Accept": "text/event-stream"}
    if api_key:
        headers["Authorization"] = f"Bearer {api_key}"
    req = urllib.request.Request(url, data=json.dumps(body).encode(), headers=headers, method="POST")
    try:
        r = urllib.request.urlopen(req, timeout=timeout)
    except urllib.error.HTTPError as e:
        try:
            msg = json.loads(e.read()).get("error", "")
        except Exception:
            msg = ""
        raise HTTPError(e.code, msg)
    with r:
        name = None
        for raw in r:
            line = raw.decode().rstrip("\r\n")
            if line.startswith("event: "):
                name = line[7:]
            elif line.startswith("data: "):
                yield name, line[6:]
                name = None


class Raw:
    """A handler's answer sent as bytes (``application/octet-stream`` unless told otherwise)."""

    def __init__(self, body: bytes, ctype: str = "application/octet-stream"):
        self.body, self.ctype = body, ctype


def fetch_bytes(url: str, api_key: Optional[str] = None, timeout: float = 600.0) -> bytes:
    req = urllib.request.Request(url, headers={"Authorization": f"Bearer {api_key}"} if api_key else {})
    try:
        with urllib.request.urlopen(req, timeout=timeout) as r:
            return r.read()
    except urllib.error.HTTPError as e:
        raise HTTPError(e.code, e.read().decode(errors="replace")[:200])
    except (urllib.error.URLError, ConnectionError, OSError) as e:
        raise HTTPError(503, f"{url} unreachable: {e!r}")


class JsonService:
    """``svc.route("POST", "/x")(fn)``; path segments ``{name}`` capture into ``ctx.params``."""

    def __init__(self, name: str, host: str = "127.0.0.1", port: Optional[int] = None):
        self.name, self.host, self.port = name, host, port or find_free_ports(1)[0]
        self._routes: list[tuple[str, list[str], Callable]] = []
        self._srv: Optional[ThreadingHTTPServer] = None

    @property
    def address(self) -> str:
        return f"{self.host}:{self.port}"

    @property
    def url(self) -> str:
        return f"http://{self.address}"

    def route(self, method: str, path: str):
        def deco(fn):
            self._routes.append((method.upper(), path.strip("/").split("/"), fn))
            return fn
        return deco

    def _match(self, method: str, path: str):
        segs = path.split("?")[0].strip("/").split("/")
        for m, pat, fn in self._routes:
            if m != method or len(pat) != len(segs):
                continue
            params = {}
            for p, s in zip(pat, segs):
                if p.startswith("{") and p.endswith("}"):
                    params[p[1:-1]] = s
                elif p != s:
                    break
            else:
                return fn, params
        return None, {}

    def start(self):
        svc = self

        class H(BaseHTTPRequestHandler):
            protocol_version = "HTTP/1.1"

            def log_message(self, *a):
                pass

            def _key(self):
                a = self.headers.get("Authorization", "")
                return a[7:].strip() if a.lower().startswith("bearer ") else self.headers.get("x-api-key")

            def _reply(self, code, obj):
                b = json.dumps(obj).encode()
                self.send_response(code)
                self.send_header("Content-Type", "application/json")
                self.send_header("Content-Length", str(len(b)))
                self.end_headers()
                self.wfile.write(b)

            def _stream(self, events):
                self.send_response(200)
                self.send_header("Content-Type", "text/event-stream")
                self.send_header("Cache-Control", "no-cache")
                self.send_header("Transfer-Encoding", "chunked")
                self.end_headers()
                for e in events:
                    if isinstance(e, tuple) and e[0] is not None:
                        data = f"event: {e[0]}\ndata: {e[1] if isinstance(e[1], str) else json.dumps(e[1])}\n\n"
                    else:
                        if isinstance(e, tuple):
                            e = e[1]
                        data = f"data: {e if isinstance(e, str) else json.dumps(e)}\n\n"
                    raw = data.encode()
                    self.wfile.write(f"{len(raw):x}\r\n".encode() + raw + b"\r\n")
                    self.wfile.flush()
                self.wfile.write(b"0\r\n\r\n")

            def _handle(self, method):
                fn, params = svc._match(method, self.path)
                if fn is None:
                    return self._reply(404, {"error": f"no route {method} {self.path}"})
                try:
                    n = int(self.headers.get("Content-Length", "0"))
                    body = json.loads(self.rfile.read(n)) if n else {}
                    res = fn(body, RequestCtx(self._key(), self.path, params, self.headers))
                    if isinstance(res, SSE):
                        return self._stream(res.events)
                    if isinstance(res, Raw):
                        self.send_response(200)
                        self.send_header("Content-Type", res.ctype)
                        self.send_header("Content-Length", str(len(res.body)))
                        self.end_headers()
                        self.wfile.write(res.body)
                        return
                    if isinstance(res, tuple):
                        return self._reply(res[0], res[1])
                    return self._reply(200, res if res is not None else {"ok": True})
                except HTTPError as e:
                    self._reply(e.status, {"error": e.message})
                except (KeyError, ValueError, TypeError) as e:
                    self._reply(400, {"error": repr(e)})
                except Exception as e:
                    logger.error("%s %s %s failed: %r", svc.name, method, self.path, e)
                    self._reply(500, {"error": repr(e)})

            def do_GET(self):
                self._handle("GET")

            def do_POST(self):
                self._handle("POST")

            def do_DELETE(self):
                self._handle("DELETE")

        self._srv = ThreadingHTTPServer((self.host, self.port), H)
        self._srv.daemon_threads = True
        self._srv.request_queue_size = 512
        threading.Thread(target=self._srv.serve_forever, daemon=True, name=f"{self.name}-http").start()
        return self

    def stop(self):
        if self._srv is not None:
            self._srv.shutdown()
            self._srv.server_close()
            self._srv = None


def call(url: str, body: Optional[dict] = None, method: Optional[str] = None, api_key: Optional[str] = None, timeout: float = 600.0,
         retries: int = 1) -> dict:
    """JSON request; raises :class:`HTTPError` for 4xx/5xx answers."""
    data = json.dumps(body).encode() if body is not None else None
    headers = {"Content-Type": "application/json"}
    if api_key:
        headers["Authorization"] = f"Bearer {api_key}"
    last: Optional[BaseException] = None
    for attempt in range(retries):
        req = urllib.request.Request(url, data=data, headers=headers, method=method or ("POST" if data is not None else "GET"))
        try:
            with urllib.request.urlopen(req, timeout=timeout) as r:
                return json.loads(r.read() or b"{}")
        except urllib.error.HTTPError as e:
            try:
                msg = json.loads(e.read()).get("error", "")
            except Exception:
                msg = ""
            if e.code < 500 or attempt + 1 == retries:
                raise HTTPError(e.code, msg)
            last = e
        except (urllib.error.URLError, ConnectionError, OSError) as e:
            last = e
        time.sleep(0.2 * (attempt + 1))
    raise HTTPError(503, f"{url} unreachable: {last!r}")
