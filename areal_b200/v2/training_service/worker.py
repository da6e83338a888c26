"""Training-service worker: one train engine behind an HTTP API. Calls are executed by one
engine thread in arrival order (collectives stay aligned across workers). Reference:
``areal/v2/training_service/worker/{app.py, engine.py}``.

Routes (bodies and answers use the RPC value envelope for tensors / dataclasses):
    GET  /health
    POST /ppo/actor/compute_logp | compute_advantages | update
    POST /ppo/critic/compute_values | update
    POST /sft/train | /sft/eval      POST /rw/train | /rw/eval      POST /dpo/train | /dpo/eval
    POST /forward        {batch, output}
    POST /save | /load   {meta}
    POST /set_version    {version}        POST /step_lr_scheduler
    GET  /export_stats   GET /version
"""
from __future__ import annotations

import queue
import threading
from concurrent.futures import Future
from typing import Any, Optional

from ...infra.rpc.serialization import deserialize_value, serialize_value
from ..common import HTTPError, JsonService

_ROUTES = {
    "/ppo/actor/compute_logp": "compute_logp", "/ppo/actor/compute_advantages": "compute_advantages", "/ppo/actor/update": "ppo_update",
    "/ppo/critic/compute_values": "compute_values", "/ppo/critic/update": "ppo_update",
    "/sft/train": "train_lm", "/sft/eval": "evaluate_lm", "/rw/train": "train_rw", "/rw/eval": "evaluate_rw",
    "/dpo/train": "train_dpo", "/dpo/eval": "evaluate_dpo",
}


class TrainingWorker:
    def __init__(self, engine, host: str = "127.0.0.1", port: Optional[int] = None):
        self.engine = engine
        self._q: "queue.Queue" = queue.Queue()
        self._thread = threading.Thread(target=self._loop, daemon=True, name="train-worker-engine")
        self._thread.start()
        self.svc = JsonService("training_worker", host, port)
        self._install()

    def _loop(self):
        while True:
            fn, fut = self._q.get()
            if fn is None:
                return
            try:
                fut.set_result(fn())
            except BaseException as e:
                fut.set_exception(e)

    def _run(self, fn):
        fut: Future = Future()
        self._q.put((fn, fut))
        return fut.result()

    def _install(self):
        svc, eng = self.svc, self.engine

        @svc.route("GET", "/health")
        def health(body, ctx):
            return {"status": "ok", "engine": type(eng).__name__, "version": eng.get_version()}

        @svc.route("GET", "/topology")
        def topology(body, ctx):
            return self.topology()

        @svc.route("GET", "/version")
        def version(body, ctx):
            return {"version": eng.get_version()}

        @svc.route("GET", "/export_stats")
        def stats(body, ctx):
            return {"stats": self._run(eng.export_stats)}

        def make(method):
            def fn(body, ctx):
                if not hasattr(eng, method):
                    raise HTTPError(404, f"engine {type(eng).__name__} has no '{method}'")
                args = deserialize_value(body)
                batch = args.pop("batch")
                res = self._run(lambda: getattr(eng, method)(batch, **args))
                return {"result": serialize_value(res)}
            return fn
        for path, method in _ROUTES.items():
            svc.route("POST", path)(make(method))

        @svc.route("POST", "/forward")
        def forward(body, ctx):
            args = deserialize_value(body)
            batch = args.pop("batch")
            return {"result": serialize_value(self._run(lambda: eng.forward_batch(batch, **args)))}

        @svc.route("POST", "/save")
        def save(body, ctx):
            self._run(lambda: eng.save(deserialize_value(body)["meta"]))
            return {"ok": True}

        @svc.route("POST", "/load")
        def load(body, ctx):
            self._run(lambda: eng.load(deserialize_value(body)["meta"]))
            return {"ok": True}

        @svc.route("GET", "/weights")
        def weights(body, ctx):
            # the complete weight dictionary by parameter name (gathered over the model-parallel ranks by the engine),
            # serialised once per version: every inference worker of a pair pulls the same bytes
            import io

            import torch

            from ..common import Raw

            v = eng.get_version()
            cached = getattr(self, "_weights_cache", None)
            if cached is None or cached[0] != v:
                w = self._run(eng.export_weights)
                buf = io.BytesIO()
                torch.save({k: t.detach().cpu() for k, t in w.items()}, buf)
                cached = self._weights_cache = (v, buf.getvalue())
            return Raw(cached[1])

        @svc.route("POST", "/set_version")
        def set_version(body, ctx):
            self._run(lambda: eng.set_version(int(body["version"])))
            return {"ok": True}

        @svc.route("POST", "/step_lr_scheduler")
        def step_lr(body, ctx):
            self._run(eng.step_lr_scheduler)
            return {"ok": True}

    def topology(self) -> dict:
        """This worker's place in the parallel layout, as its engine reports it (a single-process engine is its own
        data-parallel group of one)."""
        eng = self.engine
        g = lambda name, default: getattr(eng, name, default)      # noqa: E731
        head = eng.is_data_parallel_head() if hasattr(eng, "is_data_parallel_head") else True
        return {"address": self.address, "rank": int(g("rank", 0) or 0), "dp_rank": int(g("dp_rank", g("data_parallel_rank", 0)) or 0),
                "dp_size": int(g("dp_size", g("data_parallel_world_size", 1)) or 1), "is_dp_head": bool(head)}

    def register(self, router_address: str, heartbeat_s: float = 5.0) -> None:
        """Announces this worker to a training router and keeps the entry alive from a daemon thread."""
        from ..common import call

        call(f"http://{router_address}/register", self.topology(), retries=5)

        def beat():
            while not self._stopped.wait(heartbeat_s):
                try:
                    call(f"http://{router_address}/heartbeat", {"address": self.address})
                except Exception:  # noqa: BLE001  (the router may be restarting; the next beat tries again)
                    pass
        self._stopped = threading.Event()
        threading.Thread(target=beat, daemon=True, name="train-worker-heartbeat").start()

    def start(self):
        self.svc.start()
        return self

    def stop(self):
        self.svc.stop()
        if getattr(self, "_stopped", None) is not None:
            self._stopped.set()
        self._q.put((None, None))

    @property
    def address(self) -> str:
        return self.svc.address
