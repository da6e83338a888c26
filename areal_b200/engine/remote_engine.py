"""Client-side inference engine for rollout servers reached over HTTP.

Implements the ``InferenceEngine`` contract against one or more servers (this framework's own
``areal_b200.engine.server`` or any server speaking the same routes): server discovery
through ``name_resolve`` or explicit addresses, round-robin scheduling with request-id
affinity, interruptible ``agenerate`` (a generation aborted by a weight update is resubmitted
with the tokens produced so far; every token keeps the version that sampled it), weight-update
fan-out, pause / continue, and the workflow executor on top. Reference:
``areal/infra/remote_inf_engine.py:434-1695`` and ``areal/engine/sglang_remote.py``.
"""
from __future__ import annotations

import asyncio
import os
import subprocess
import sys
import threading
import time
import uuid
from concurrent.futures import Future, ThreadPoolExecutor
from typing import Any, Optional

from ..api.cli_args import InferenceEngineConfig
from ..api.engine_api import InferenceEngine
from ..api.io_struct import ModelRequest, ModelResponse, ParamSpec, WeightUpdateMeta
from ..utils import logging as alog
from ..utils import name_resolve, names

logger = alog.getLogger("remote_engine")


async def arequest_with_retry(session, addr: str, endpoint: str, payload: Optional[dict] = None, method: str = "POST",
                              max_retries: int = 3, timeout: float = 3600.0, retry_delay: float = 0.5) -> dict:
    """One JSON request with bounded retries on connection errors and 5xx answers."""
    import aiohttp

    last: Optional[BaseException] = None
    url = f"http://{addr}{endpoint}"
    for attempt in range(max_retries):
        try:
            async with session.request(method, url, json=payload, timeout=aiohttp.ClientTimeout(total=timeout)) as r:
                if r.status >= 500:
                    raise RuntimeError(f"{url} -> HTTP {r.status}: {(await r.text())[:500]}")
                r.raise_for_status()
                return await r.json()
        except (aiohttp.ClientConnectionError, asyncio.TimeoutError, RuntimeError) as e:
            last = e
            if attempt + 1 < max_retries:
                await asyncio.sleep(retry_delay * (attempt + 1))
    raise RuntimeError(f"request to {url} failed after {max_retries} attempts: {last!r}")


class RemoteInfEngine(InferenceEngine):
    def __init__(self, config: InferenceEngineConfig, addresses: Optional[list[str]] = None, backend: Optional[str] = None):
        """``backend``: wire format of the servers (``native`` | ``sglang`` | ``vllm``, see ``remote_backends.py``);
        default: ``config.backend`` if it names one, else this repository's server."""
        from .remote_backends import BACKENDS, get_backend

        self.config = config
        name = backend if backend is not None else (getattr(config, "backend", "") or "")
        self.backend = get_backend(name.split(":")[0] if name.split(":")[0].lower() in BACKENDS else "native")
        self.addresses: list[str] = list(addresses or [])
        self._version = 0
        self._rr = 0
        self._rid_to_addr: dict[str, str] = {}
        self._rid_order: list[str] = []
        self._inflight: dict[str, int] = {}          # address -> requests of this client being served there
        self._lock = threading.Lock()
        self._executor = None
        self._paused = threading.Event()
        self._pool = ThreadPoolExecutor(max_workers=8, thread_name_prefix="remote-engine")
        self._sessions: dict[int, Any] = {}
        self._server_procs: list[subprocess.Popen] = []
        self._initialized = False

    # ------------------------------------------------------------------ lifecycle
    def initialize(self, addr: Optional[Any] = None, train_data_parallel_size: int = 1, start_executor: bool = True, **kwargs):
        if addr:
            self.addresses = [addr] if isinstance(addr, str) else list(addr)
        if not self.addresses and os.environ.get("AREAL_LLM_SERVER_ADDRS"):
            self.addresses = os.environ["AREAL_LLM_SERVER_ADDRS"].split(",")
        if not self.addresses:
            key = names.gen_servers(self.config.experiment_name or "", self.config.trial_name or "")
            deadline = time.monotonic() + self.config.setup_timeout
            while time.monotonic() < deadline:
                self.addresses = sorted(set(name_resolve.get_subtree(key)))
                if self.addresses:
                    break
                time.sleep(0.5)
        if not self.addresses:
            raise RuntimeError("no inference server address (argument, AREAL_LLM_SERVER_ADDRS or name_resolve)")
        self._wait_healthy()
        if start_executor:
            from ..rollout.executor import WorkflowExecutor

            self._executor = WorkflowExecutor(self.config, self, dp_world_size=train_data_parallel_size).initialize()
        self._initialized = True
        return self

    @property
    def initialized(self) -> bool:
        return self._initialized

    def _wait_healthy(self):
        import urllib.request

        deadline = time.monotonic() + self.config.setup_timeout
        for a in self.addresses:
            while True:
                try:
                    with urllib.request.urlopen(f"http://{a}/health", timeout=2) as r:
                        if r.status == 200:
                            break
                except OSError:
                    pass
                if time.monotonic() > deadline:
                    raise TimeoutError(f"inference server {a} not healthy after {self.config.setup_timeout}s")
                time.sleep(0.2)

    def destroy(self):
        if self._executor is not None:
            self._executor.destroy()
            self._executor = None
        self.teardown_server()
        self._pool.shutdown(wait=False)
        self._initialized = False

    def launch_server(self, server_args: dict[str, Any]) -> str:
        """Starts a local server process (``python -m areal_b200.engine.server``) and returns
        its address once it reports ready."""
        if self.backend.name != "native" or "cmd" in server_args:
            return self._launch_external_server(dict(server_args))
        cmd = [sys.executable, "-m", "areal_b200.engine.server"]
        for k, v in server_args.items():
            cmd += [f"--{k.replace('_', '-')}", str(v)]
        p = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, start_new_session=True)
        self._server_procs.append(p)
        deadline = time.monotonic() + self.config.setup_timeout
        addr = None
        while time.monotonic() < deadline:
            line = p.stdout.readline()
            if not line:
                if p.poll() is not None:
                    raise RuntimeError(f"inference server exited with code {p.returncode}")
                continue
            if line.startswith("INFER_SERVER_READY"):
                addr = line.split()[1]
                break
        if addr is None:
            raise TimeoutError("inference server did not become ready")
        threading.Thread(target=lambda: [None for _ in p.stdout], daemon=True).start()  # keep draining the pipe
        self.addresses.append(addr)
        return addr

    def _launch_external_server(self, server_args: dict[str, Any]) -> str:
        """An SGLang / vLLM server as a child process: ``server_args`` are the server's own flags (``host`` and ``port``
        among them; see ``SGLangConfig.build_args`` / ``vLLMConfig.build_args``) or carry a ready command line under
        ``cmd``. Ready when its health route answers. Reference: ``areal/engine/sglang_remote.py:394-420``,
        ``areal/engine/vllm_remote.py`` (``launch_server``)."""
        import urllib.request

        from ..api.cli_args import server_cmd
        from ..utils.network import find_free_ports

        host = server_args.get("host") or "127.0.0.1"
        port = server_args.get("port") or find_free_ports(1)[0]
        cmd = server_args.pop("cmd", None)
        if cmd is None:
            server_args.update(host=host, port=port)
            module = {"sglang": "sglang.launch_server", "vllm": "vllm.entrypoints.openai.api_server"}[self.backend.name]
            cmd = server_cmd(module, server_args)
        p = subprocess.Popen([str(c) for c in cmd], stdout=subprocess.DEVNULL, stderr=subprocess.STDOUT, start_new_session=True)
        self._server_procs.append(p)
        from ..utils.network import format_hostport

        addr = format_hostport(host, port)
        deadline = time.monotonic() + self.config.setup_timeout
        while True:
            if p.poll() is not None:
                raise RuntimeError(f"{self.backend.name} server exited with code {p.returncode}")
            try:
                with urllib.request.urlopen(f"http://{addr}{self.backend.health_endpoint}", timeout=2) as r:
                    if r.status == 200:
                        break
            except OSError:
                pass
            if time.monotonic() > deadline:
                raise TimeoutError(f"{self.backend.name} server {addr} not healthy after {self.config.setup_timeout}s")
            time.sleep(0.2)
        self.addresses.append(addr)
        return addr

    def teardown_server(self):
        for p in self._server_procs:
            if p.poll() is None:
                p.terminate()
                try:
                    p.wait(timeout=10)
                except subprocess.TimeoutExpired:
                    p.kill()
        self._server_procs.clear()

    # ------------------------------------------------------------------ scheduling
    def choose_server(self, rid: Optional[str] = None) -> str:
        with self._lock:
            if rid is not None and rid in self._rid_to_addr:
                return self._rid_to_addr[rid]          # KV-cache affinity for resumed / multi-turn requests
            if getattr(self.config, "schedule_policy", "round_robin") in ("least_requests", "least_loaded") and self._inflight:
                # the server with the fewest requests of this client in flight (ties: the earliest in the list)
                a = min(self.addresses, key=lambda x: (self._inflight.get(x, 0), self.addresses.index(x)))
            else:
                a = self.addresses[self._rr % len(self.addresses)]
            self._rr += 1
            if rid is not None:
                self._rid_to_addr[rid] = a
                self._rid_order.append(rid)
                if len(self._rid_order) > 1 << 16:
                    for old in self._rid_order[: 1 << 15]:
                        self._rid_to_addr.pop(old, None)
                    del self._rid_order[: 1 << 15]
            return a

    async def _session(self):
        import aiohttp

        loop = asyncio.get_running_loop()
        s = self._sessions.get(id(loop))
        if s is None or s.closed:
            s = aiohttp.ClientSession(connector=aiohttp.TCPConnector(limit=0))
            self._sessions[id(loop)] = s
        return s

    # ------------------------------------------------------------------ generation
    async def agenerate(self, req: ModelRequest) -> ModelResponse:
        g = req.gconfig
        if g.n_samples != 1:
            raise ValueError("agenerate serves one sample per request; workflows fan out n_samples themselves")
        prompt = list(req.input_ids)
        budget = min(g.max_new_tokens, g.max_tokens - len(prompt))
        if budget <= 0:
            raise ValueError(f"prompt of {len(prompt)} tokens leaves no room under max_tokens={g.max_tokens}")
        out_tok: list[int] = []
        out_lp: list[float] = []
        out_ver: list[int] = []
        stop = "abort"
        t0 = time.perf_counter()
        ttft = float("inf")
        addr = self.choose_server(req.rid)
        session = await self._session()
        with self._lock:
            self._inflight[addr] = self._inflight.get(addr, 0) + 1
        try:
            return await self._generate_on(addr, session, req, g, prompt, budget, out_tok, out_lp, out_ver, stop, t0, ttft)
        finally:
            with self._lock:
                self._inflight[addr] = max(0, self._inflight.get(addr, 1) - 1)

    async def _generate_on(self, addr, session, req, g, prompt, budget, out_tok, out_lp, out_ver, stop, t0, ttft) -> ModelResponse:
        while stop not in ("stop", "length", "tool_calls") and len(out_tok) < budget:
            while self._paused.is_set():
                await asyncio.sleep(0.01)
            version_sent = self._version          # a weight update may land while the request is in flight
            hr = self.backend.build_generation(req.rid, prompt + out_tok, g, budget, len(out_tok))
            r = await arequest_with_retry(session, addr, hr.endpoint, hr.payload, method=hr.method, max_retries=self.config.request_retries,
                                          timeout=self.config.request_timeout)
            res = self.backend.parse_generation(r)
            seg = res.tokens
            if seg and ttft == float("inf"):
                ttft = time.perf_counter() - t0
            out_tok += seg
            out_lp += res.logprobs if len(res.logprobs) == len(seg) else [0.0] * len(seg)
            # servers that do not tag tokens: the version that was current when the request left served it
            out_ver += res.versions or [version_sent] * len(seg)
            stop = res.stop_reason
            if stop == "abort" and not seg:
                await asyncio.sleep(0.02)     # server is paused for a weight update
        if stop == "abort":
            stop = "length"
        lat = time.perf_counter() - t0
        return ModelResponse(input_tokens=prompt, output_tokens=out_tok, output_logprobs=out_lp, output_versions=out_ver,
                             stop_reason=stop, latency=lat, ttft=ttft, tokenizer=req.tokenizer)

    # ------------------------------------------------------------------ control fan-out
    def _fanout(self, endpoint: str, payload: Optional[dict] = None, timeout: float = 3600.0) -> list[dict]:
        import json
        import urllib.request

        def one(a):
            req = urllib.request.Request(f"http://{a}{endpoint}", data=json.dumps(payload or {}).encode(),
                                         headers={"Content-Type": "application/json"})
            with urllib.request.urlopen(req, timeout=timeout) as r:
                return json.loads(r.read())
        return list(self._pool.map(one, self.addresses))

    def _fanout_future(self, endpoint: str, payload_fn, after=None) -> Future:
        fut: Future = Future()

        def run():
            try:
                import json
                import urllib.request

                def one(ia):
                    i, a = ia
                    req = urllib.request.Request(f"http://{a}{endpoint}", data=json.dumps(payload_fn(i)).encode(),
                                                 headers={"Content-Type": "application/json"})
                    with urllib.request.urlopen(req, timeout=self.config.request_timeout) as r:
                        return json.loads(r.read())
                res = list(self._pool.map(one, enumerate(self.addresses)))
                if after:
                    after()
                fut.set_result(res)
            except BaseException as e:
                fut.set_exception(e)
        threading.Thread(target=run, daemon=True).start()
        return fut

    def _requests_future(self, request_fns: list, after=None) -> Future:
        """Sends, one after the other, the requests ``request_fns[k](server index)`` to every server."""
        fut: Future = Future()

        def run():
            try:
                out = []
                for fn in request_fns:
                    first = fn(0)
                    out = self._fanout_future(first.endpoint, lambda i, fn=fn: fn(i).payload).result()
                if after:
                    after()
                fut.set_result(out)
            except BaseException as e:
                fut.set_exception(e)
        threading.Thread(target=run, daemon=True).start()
        return fut

    def set_version(self, version: int) -> None:
        self._version = version
        hr = self.backend.set_version(version)
        if hr is not None:
            self._fanout(hr.endpoint, hr.payload)

    def get_version(self) -> int:
        return self._version

    def pause_generation(self):
        self._paused.set()
        self._fanout(self.backend.pause_endpoint)
        grace = float(getattr(self.config, "pause_grace_period", 0.0) or 0.0)
        if grace > 0:
            time.sleep(grace)          # lets requests that were already on their way to a server reach it and be aborted there

    def continue_generation(self):
        self._fanout(self.backend.continue_endpoint)
        self._paused.clear()

    def update_weights_from_disk(self, meta: WeightUpdateMeta) -> Future:
        def done():
            if meta.version is not None:
                self._version = meta.version
        return self._requests_future([lambda i, r=r: r for r in self.backend.disk_update(meta)], done)

    def init_weights_update_group(self, meta: WeightUpdateMeta) -> Future:
        n = len(self.addresses)
        return self._requests_future([lambda i: self.backend.init_group(meta, i, n)])

    def update_weights_from_distributed(self, meta: WeightUpdateMeta, param_specs: list[ParamSpec]) -> Future:
        def done():
            if meta.version is not None:
                self._version = meta.version
        return self._requests_future([lambda i, r=r: r for r in self.backend.distributed_update(meta, param_specs)], done)

    def update_weights_from_tensors(self, named_tensors, meta: Optional[WeightUpdateMeta] = None) -> Future:
        raise NotImplementedError("tensors cannot be handed to another process; use disk, xccl or p2p weight updates")

    def offload(self, tags: Optional[list[str]] = None):
        self._fanout(self.backend.offload_endpoint, {"tags": tags})

    def onload(self, tags: Optional[list[str]] = None):
        self._fanout(self.backend.onload_endpoint, {"tags": tags})

    # ------------------------------------------------------------------ executor passthrough
    def submit(self, data, workflow=None, workflow_kwargs=None, should_accept_fn=None, task_id=None, is_eval=False) -> int:
        return self._executor.submit(data, workflow, workflow_kwargs, should_accept_fn, task_id, is_eval)

    def wait(self, count, timeout=None, raise_timeout=True):
        return self._executor.wait(count, timeout, raise_timeout)

    def wait_for_task(self, task_id, timeout=None, raise_timeout=True):
        return self._executor.wait_for_task(task_id, timeout, raise_timeout)

    def rollout_batch(self, data, workflow=None, workflow_kwargs=None, should_accept_fn=None):
        return self._executor.rollout_batch(data, workflow, workflow_kwargs, should_accept_fn)

    def prepare_batch(self, dataloader, workflow=None, workflow_kwargs=None, should_accept_fn=None, dynamic_bs=False):
        return self._executor.prepare_batch(dataloader, workflow, workflow_kwargs, should_accept_fn, dynamic_bs)

    def pause(self):
        if self._executor is not None:
            self._executor.pause()

    def resume(self):
        if self._executor is not None:
            self._executor.resume()

    def export_stats(self) -> dict[str, float]:
        return {}


RemoteNativeEngine = RemoteInfEngine
