"""Code execution on another host.

``SandboxServer`` exposes a :class:`LocalSandbox` behind HTTP (``POST /run`` with a bearer key, a bound on
concurrent runs, per-request limits capped by the server's own); ``RemoteSandbox`` is the client with the interface
of ``LocalSandbox`` (``run`` / ``arun``), so rollout workflows and reward functions take either. ``DaytonaRunner``
gives the same interface over a Daytona cloud sandbox when its SDK is installed (the hosted backend of the
reference, ``areal/infra/sandbox/runner.py:102-371``); without the SDK it says so on construction.
"""
from __future__ import annotations

import asyncio
import threading
from typing import Optional

from ...v2.common import HTTPError, JsonService, call
from .local import ExecResult, LocalSandbox, SandboxConfig


class SandboxServer:
    def __init__(self, config: Optional[SandboxConfig] = None, host: str = "127.0.0.1", port: Optional[int] = None,
                 api_key: Optional[str] = None, max_concurrent: int = 8):
        self.cfg = config or SandboxConfig()
        self.api_key = api_key
        self.svc = JsonService("sandbox", host, port)
        self._slots = threading.BoundedSemaphore(max_concurrent)
        self.runs = 0
        svc = self.svc

        @svc.route("GET", "/health")
        def health(body, ctx):
            return {"status": "ok", "runs": self.runs, "timeout_s": self.cfg.timeout_s}

        @svc.route("POST", "/run")
        def run(body, ctx):
            if self.api_key and ctx.api_key != self.api_key:
                raise HTTPError(401, "sandbox key required")
            code = body.get("code")
            if not isinstance(code, str):
                raise HTTPError(400, "'code' (a string) is required")
            # a request may ask for less than the server allows, never for more
            c = SandboxConfig(timeout_s=min(float(body.get("timeout_s", self.cfg.timeout_s)), self.cfg.timeout_s),
                              cpu_time_s=self.cfg.cpu_time_s, memory_mb=min(int(body.get("memory_mb", self.cfg.memory_mb)), self.cfg.memory_mb),
                              max_output_bytes=self.cfg.max_output_bytes, python=self.cfg.python, env=dict(self.cfg.env),
                              allow_network_env=self.cfg.allow_network_env)
            if not self._slots.acquire(timeout=float(body.get("queue_timeout_s", 60.0))):
                raise HTTPError(503, "sandbox is busy")
            try:
                r = LocalSandbox(c).run(code, stdin=body.get("stdin", ""), files=body.get("files"))
                self.runs += 1
            finally:
                self._slots.release()
            return {"stdout": r.stdout, "stderr": r.stderr, "returncode": r.returncode, "timed_out": r.timed_out, "seconds": r.seconds}

    def start(self):
        self.svc.start()
        return self

    def stop(self):
        self.svc.stop()

    @property
    def address(self) -> str:
        return self.svc.address


class RemoteSandbox:
    def __init__(self, address: str, api_key: Optional[str] = None, timeout_s: Optional[float] = None, retries: int = 2):
        self.address, self.api_key, self.timeout_s, self.retries = address, api_key, timeout_s, retries

    def run(self, code: str, stdin: str = "", files: Optional[dict[str, str]] = None) -> ExecResult:
        body = {"code": code, "stdin": stdin, "files": files or {}}
        if self.timeout_s is not None:
            body["timeout_s"] = self.timeout_s
        r = call(f"http://{self.address}/run", body, api_key=self.api_key, timeout=(self.timeout_s or 60.0) + 90.0, retries=self.retries)
        return ExecResult(r["stdout"], r["stderr"], int(r["returncode"]), bool(r["timed_out"]), float(r["seconds"]))

    async def arun(self, code: str, stdin: str = "", files: Optional[dict[str, str]] = None) -> ExecResult:
        return await asyncio.get_running_loop().run_in_executor(None, self.run, code, stdin, files)


class DaytonaRunner:
    """Same interface over a Daytona cloud sandbox (one sandbox per runner, created on first use, deleted by
    ``close()``). Needs the ``daytona`` package and credentials in the environment; neither ships with this
    repository."""

    def __init__(self, language: str = "python", timeout_s: float = 60.0, **create_kwargs):
        try:
            import daytona  # noqa: F401
        except ImportError as e:
            raise ImportError("the Daytona backend needs the 'daytona' package (pip install daytona) and DAYTONA_API_KEY; "
                              "use LocalSandbox or RemoteSandbox otherwise") from e
        self._sdk = daytona
        self.language, self.timeout_s, self.create_kwargs = language, timeout_s, create_kwargs
        self._sandbox = None
        self._client = None

    def _ensure(self):
        if self._sandbox is None:
            self._client = self._sdk.Daytona()
            self._sandbox = self._client.create(self._sdk.CreateSandboxFromSnapshotParams(language=self.language, **self.create_kwargs))
        return self._sandbox

    def run(self, code: str, stdin: str = "", files: Optional[dict[str, str]] = None) -> ExecResult:
        import time

        sb = self._ensure()
        for name, content in (files or {}).items():
            sb.fs.upload_file(content.encode(), name)
        t0 = time.monotonic()
        try:
            resp = sb.process.code_run(code, timeout=int(self.timeout_s))
            return ExecResult(resp.result or "", "", int(resp.exit_code), False, time.monotonic() - t0)
        except Exception as e:      # the SDK raises on time-outs and transport errors alike
            return ExecResult("", repr(e), -1, "timeout" in repr(e).lower(), time.monotonic() - t0)

    async def arun(self, code: str, stdin: str = "", files: Optional[dict[str, str]] = None) -> ExecResult:
        return await asyncio.get_running_loop().run_in_executor(None, self.run, code, stdin, files)

    def close(self) -> None:
        if self._sandbox is not None and self._client is not None:
            try:
                self._client.delete(self._sandbox)
            finally:
                self._sandbox = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()
