"""The data service: datasets hosted by worker processes next to storage, one gateway address for the trainers.

    DataWorker    holds the datasets it was told to load and serves samples by index
    DataRouter    registry of live workers (register / unregister / health polling)
    DataGateway   registers a dataset on every worker and hands out a token for it; fetches fan out to the
                  workers that own the requested indices (index i lives on worker i mod n) and come back in
                  request order; epoch advance, state save / load and status are broadcast
    DataController starts the three roles (threads of this process, or worker addresses given by a scheduler)
                  and returns :class:`rdataset.RDataset` handles bound to a token

Routes and payloads follow the reference (``areal/infra/data_service/{worker,router,gateway}/app.py``,
``controller/controller.py``); the services are the stdlib JSON scaffold of ``v2/common.py``.
"""
from __future__ import annotations

import concurrent.futures as cf
import json
import os
import secrets
import threading
import time
from typing import Any, Callable, Optional

from ...utils import logging as alog
from ...utils.dynamic_import import import_from_string
from ...v2.common import HTTPError, JsonService, call
from ..rpc.serialization import deserialize_value, serialize_value

logger = alog.getLogger("data_service")


def _admin(ctx, key: Optional[str]) -> None:
    if key and ctx.api_key != key:
        raise HTTPError(401, "admin key required")


class _Hosted:
    def __init__(self, dataset, spec: dict):
        self.dataset, self.spec = dataset, spec
        self.epoch = 0
        self.served = 0
        self.lock = threading.Lock()


class DataWorker:
    def __init__(self, host: str = "127.0.0.1", port: Optional[int] = None, admin_key: Optional[str] = None, rank: int = 0, world: int = 1):
        self.svc = JsonService("data_worker", host, port)
        self.admin_key, self.rank, self.world = admin_key, rank, world
        self.datasets: dict[str, _Hosted] = {}
        self._lock = threading.Lock()
        svc = self.svc

        def need(did: str) -> _Hosted:
            h = self.datasets.get(did)
            if h is None:
                raise HTTPError(404, f"dataset '{did}' is not loaded on this worker")
            return h

        @svc.route("GET", "/health")
        def health(body, ctx):
            return {"status": "ok", "rank": self.rank, "datasets": {k: len(v.dataset) for k, v in self.datasets.items()}}

        @svc.route("POST", "/datasets/load")
        def load(body, ctx):
            _admin(ctx, self.admin_key)
            did = body["dataset_id"]
            if did in self.datasets:
                return {"dataset_id": did, "len": len(self.datasets[did].dataset), "already_loaded": True}
            if body.get("factory"):
                ds = import_from_string(body["factory"])(**(body.get("kwargs") or {}))
            else:
                from ...dataset import get_custom_dataset

                tok = import_from_string(body["tokenizer"])(**(body.get("tokenizer_kwargs") or {})) if body.get("tokenizer") else None
                ds = get_custom_dataset(body["path"], type=body.get("type", "rl"), split=body.get("split", "train"), tokenizer=tok,
                                        max_length=body.get("max_length"), **(body.get("kwargs") or {}))
            with self._lock:
                self.datasets[did] = _Hosted(ds, {k: v for k, v in body.items() if k != "dataset_id"})
            return {"dataset_id": did, "len": len(ds)}

        @svc.route("POST", "/v1/samples/fetch")
        def fetch(body, ctx):
            h = need(body["dataset_id"])
            idx = body["indices"]
            n = len(h.dataset)
            if any((not isinstance(i, int)) or i < 0 or i >= n for i in idx):
                raise HTTPError(400, "index out of range")
            with h.lock:
                h.served += len(idx)
            return {"samples": [serialize_value(h.dataset[i]) for i in idx]}

        @svc.route("POST", "/datasets/unload")
        def unload(body, ctx):
            _admin(ctx, self.admin_key)
            with self._lock:
                gone = self.datasets.pop(body["dataset_id"], None)
            return {"unloaded": gone is not None}

        @svc.route("POST", "/epoch/reset")
        def epoch(body, ctx):
            _admin(ctx, self.admin_key)
            h = need(body["dataset_id"])
            with h.lock:
                h.epoch = int(body.get("epoch", h.epoch + 1))
                if hasattr(h.dataset, "set_epoch"):
                    h.dataset.set_epoch(h.epoch)
            return {"epoch": h.epoch}

        @svc.route("POST", "/state/save")
        def save(body, ctx):
            _admin(ctx, self.admin_key)
            h = need(body["dataset_id"])
            os.makedirs(body["path"], exist_ok=True)
            fn = os.path.join(body["path"], f"data_worker_{self.rank}_{body['dataset_id']}.json")
            with h.lock, open(fn, "w") as f:
                json.dump({"epoch": h.epoch, "served": h.served, "spec": h.spec}, f)
            return {"path": fn}

        @svc.route("POST", "/state/load")
        def load_state(body, ctx):
            _admin(ctx, self.admin_key)
            h = need(body["dataset_id"])
            fn = os.path.join(body["path"], f"data_worker_{self.rank}_{body['dataset_id']}.json")
            if not os.path.exists(fn):
                raise HTTPError(404, f"no saved state at {fn}")
            with open(fn) as f:
                st = json.load(f)
            with h.lock:
                h.epoch, h.served = int(st["epoch"]), int(st["served"])
                if hasattr(h.dataset, "set_epoch"):
                    h.dataset.set_epoch(h.epoch)
            return {"epoch": h.epoch, "served": h.served}

        @svc.route("DELETE", "/data/clear")
        def clear(body, ctx):
            _admin(ctx, self.admin_key)
            with self._lock:
                n = len(self.datasets)
                self.datasets.clear()
            return {"cleared": n}

    def start(self):
        self.svc.start()
        return self

    def stop(self):
        self.svc.stop()

    @property
    def address(self) -> str:
        return self.svc.address


class DataRouter:
    def __init__(self, host: str = "127.0.0.1", port: Optional[int] = None, admin_key: Optional[str] = None, poll_interval_s: float = 0.0):
        self.svc = JsonService("data_router", host, port)
        self.admin_key = admin_key
        self.workers: list[str] = []
        self.healthy: dict[str, bool] = {}
        self._rr = 0
        self._lock = threading.Lock()
        self._stop = threading.Event()
        self._poll_interval = poll_interval_s
        svc = self.svc

        @svc.route("GET", "/health")
        def health(body, ctx):
            return {"status": "ok", "workers": len(self.workers)}

        @svc.route("POST", "/register")
        def register(body, ctx):
            _admin(ctx, self.admin_key)
            with self._lock:
                if body["address"] not in self.workers:
                    self.workers.append(body["address"])
                self.healthy[body["address"]] = True
            return {"workers": list(self.workers)}

        @svc.route("POST", "/unregister")
        def unregister(body, ctx):
            _admin(ctx, self.admin_key)
            with self._lock:
                if body["address"] in self.workers:
                    self.workers.remove(body["address"])
                self.healthy.pop(body["address"], None)
            return {"workers": list(self.workers)}

        @svc.route("POST", "/route")
        def route(body, ctx):
            _admin(ctx, self.admin_key)
            with self._lock:
                live = [w for w in self.workers if self.healthy.get(w, False)]
                if not live:
                    raise HTTPError(503, "no healthy data worker")
                self._rr += 1
                return {"address": live[self._rr % len(live)]}

        @svc.route("GET", "/workers")
        def workers(body, ctx):
            _admin(ctx, self.admin_key)
            return {"workers": [{"address": w, "healthy": self.healthy.get(w, False)} for w in self.workers]}

    def check_health(self) -> dict:
        for w in list(self.workers):
            try:
                ok = call(f"http://{w}/health", timeout=3.0).get("status") == "ok"
            except HTTPError:
                ok = False
            self.healthy[w] = ok
        return dict(self.healthy)

    def _poll(self):
        while not self._stop.wait(self._poll_interval):
            self.check_health()

    def start(self):
        self.svc.start()
        if self._poll_interval > 0:
            threading.Thread(target=self._poll, daemon=True, name="data-router-health").start()
        return self

    def stop(self):
        self._stop.set()
        self.svc.stop()

    @property
    def address(self) -> str:
        return self.svc.address


class DataGateway:
    def __init__(self, router_addr: str, host: str = "127.0.0.1", port: Optional[int] = None, admin_key: Optional[str] = None,
                 timeout_s: float = 120.0):
        self.svc = JsonService("data_gateway", host, port)
        self.router, self.admin_key, self.timeout = router_addr, admin_key, timeout_s
        self.tokens: dict[str, str] = {}              # dataset token -> dataset id
        self.meta: dict[str, dict] = {}
        self._pool = cf.ThreadPoolExecutor(max_workers=16, thread_name_prefix="data-gw")
        self._lock = threading.Lock()
        self.shutdown_requested = threading.Event()
        svc = self.svc

        def dataset_of(ctx) -> str:
            did = self.tokens.get(ctx.api_key or "")
            if did is None:
                raise HTTPError(401, "unknown dataset token")
            return did

        @svc.route("GET", "/health")
        def health(body, ctx):
            return {"status": "ok", "datasets": len(self.meta)}

        @svc.route("POST", "/v1/datasets/register")
        def register(body, ctx):
            _admin(ctx, self.admin_key)
            did = body.get("dataset_id") or "ds-" + secrets.token_hex(6)
            res = self._broadcast("/datasets/load", {**body, "dataset_id": did})
            lens = {r["len"] for r in res}
            if len(lens) != 1:
                raise HTTPError(500, f"workers disagree on the dataset length: {sorted(lens)}")
            token = "sk-data-" + secrets.token_hex(12)
            with self._lock:
                self.tokens[token] = did
                self.meta[did] = {"len": lens.pop(), "epoch": 0, "workers": len(res)}
            return {"dataset_id": did, "api_key": token, "len": self.meta[did]["len"], "n_workers": len(res)}

        @svc.route("POST", "/v1/datasets/unregister")
        def unregister(body, ctx):
            _admin(ctx, self.admin_key)
            did = body["dataset_id"]
            self._broadcast("/datasets/unload", {"dataset_id": did})
            with self._lock:
                self.meta.pop(did, None)
                for t in [t for t, d in self.tokens.items() if d == did]:
                    del self.tokens[t]
            return {"ok": True}

        @svc.route("POST", "/v1/samples/fetch")
        def fetch(body, ctx):
            did = dataset_of(ctx)
            idx = [int(i) for i in body["indices"]]
            ws = self._workers()
            if not ws:
                raise HTTPError(503, "no data worker registered")
            by_owner: dict[int, list[int]] = {}
            for pos, i in enumerate(idx):
                by_owner.setdefault(i % len(ws), []).append(pos)

            def one(owner: int, positions: list[int]):
                r = call(f"http://{ws[owner]}/v1/samples/fetch", {"dataset_id": did, "indices": [idx[p] for p in positions]},
                         timeout=self.timeout, retries=2)
                return positions, r["samples"]
            out: list[Any] = [None] * len(idx)
            for positions, samples in self._pool.map(lambda kv: one(*kv), by_owner.items()):
                for p, s in zip(positions, samples):
                    out[p] = s
            return {"samples": out}

        @svc.route("POST", "/v1/epochs/advance")
        def advance(body, ctx):
            did = dataset_of(ctx)
            with self._lock:
                self.meta[did]["epoch"] = int(body.get("epoch", self.meta[did]["epoch"] + 1))
                e = self.meta[did]["epoch"]
            self._broadcast("/epoch/reset", {"dataset_id": did, "epoch": e})
            return {"epoch": e}

        @svc.route("POST", "/v1/state/save")
        def save(body, ctx):
            did = dataset_of(ctx)
            return {"files": [r["path"] for r in self._broadcast("/state/save", {"dataset_id": did, "path": body["path"]})]}

        @svc.route("POST", "/v1/state/load")
        def load(body, ctx):
            did = dataset_of(ctx)
            res = self._broadcast("/state/load", {"dataset_id": did, "path": body["path"]})
            with self._lock:
                self.meta[did]["epoch"] = max(r["epoch"] for r in res)
            return {"epoch": self.meta[did]["epoch"], "served": sum(r["served"] for r in res)}

        @svc.route("GET", "/v1/status")
        def status(body, ctx):
            _admin(ctx, self.admin_key)
            return {"datasets": self.meta, "workers": self._worker_table()}

        @svc.route("GET", "/v1/workers")
        def workers(body, ctx):
            _admin(ctx, self.admin_key)
            return {"workers": self._worker_table()}

        @svc.route("POST", "/v1/shutdown")
        def shutdown(body, ctx):
            _admin(ctx, self.admin_key)
            res = self._broadcast("/data/clear", None, method="DELETE")
            self.shutdown_requested.set()
            return {"cleared": sum(r["cleared"] for r in res)}

    def _worker_table(self) -> list[dict]:
        return call(f"http://{self.router}/workers", api_key=self.admin_key, timeout=10.0)["workers"]

    def _workers(self) -> list[str]:
        return [w["address"] for w in self._worker_table()]

    def _broadcast(self, path: str, body: Optional[dict], method: Optional[str] = None) -> list[dict]:
        ws = self._workers()
        if not ws:
            raise HTTPError(503, "no data worker registered")
        return list(self._pool.map(lambda a: call(f"http://{a}{path}", body, method=method, api_key=self.admin_key, timeout=self.timeout), ws))

    def start(self):
        self.svc.start()
        return self

    def stop(self):
        self.svc.stop()
        self._pool.shutdown(wait=False)

    @property
    def address(self) -> str:
        return self.svc.address


class DataController:
    """Brings the service up and registers datasets. ``worker_addrs``: workers that already run elsewhere
    (started by a scheduler with ``python -m areal_b200.infra.data_service.service worker ...``); otherwise
    ``n_workers`` workers run as threads of this process."""

    def __init__(self, n_workers: int = 1, worker_addrs: Optional[list[str]] = None, admin_key: Optional[str] = None, host: str = "127.0.0.1"):
        self.admin_key = admin_key or "adm-" + secrets.token_hex(8)
        self.host = host
        self._n, self._given = n_workers, list(worker_addrs or [])
        self.router: Optional[DataRouter] = None
        self.gateway: Optional[DataGateway] = None
        self.workers: list[DataWorker] = []

    def start(self):
        self.router = DataRouter(self.host, admin_key=self.admin_key).start()
        addrs = list(self._given)
        if not addrs:
            self.workers = [DataWorker(self.host, admin_key=self.admin_key, rank=r, world=self._n).start() for r in range(self._n)]
            addrs = [w.address for w in self.workers]
        for a in addrs:
            call(f"http://{self.router.address}/register", {"address": a}, api_key=self.admin_key)
        self.gateway = DataGateway(self.router.address, self.host, admin_key=self.admin_key).start()
        return self

    def register_dataset(self, path: Optional[str] = None, type: str = "rl", split: str = "train", factory: Optional[str] = None,
                         kwargs: Optional[dict] = None, tokenizer: Optional[str] = None, prefetch: int = 64, **extra):
        from .rdataset import RDataset

        body = {"path": path, "type": type, "split": split, "factory": factory, "kwargs": kwargs or {}, "tokenizer": tokenizer, **extra}
        r = call(f"http://{self.gateway.address}/v1/datasets/register", {k: v for k, v in body.items() if v is not None}, api_key=self.admin_key)
        return RDataset(self.gateway.address, prefetch=prefetch, token=r["api_key"], length=r["len"], dataset_id=r["dataset_id"])

    def status(self) -> dict:
        return call(f"http://{self.gateway.address}/v1/status", api_key=self.admin_key)

    def stop(self):
        for s in [self.gateway, self.router] + self.workers:
            if s is not None:
                s.stop()
        self.workers = []


def main(argv=None):
    import argparse

    ap = argparse.ArgumentParser(description="one role of the data service")
    ap.add_argument("role", choices=["worker", "router", "gateway"])
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--port", type=int, default=0)
    ap.add_argument("--admin-key", default=None)
    ap.add_argument("--router", default=None, help="router address (worker: registers itself there; gateway: required)")
    ap.add_argument("--rank", type=int, default=0)
    ap.add_argument("--world", type=int, default=1)
    a = ap.parse_args(argv)
    port = a.port or None
    if a.role == "worker":
        s = DataWorker(a.host, port, a.admin_key, a.rank, a.world).start()
        if a.router:
            call(f"http://{a.router}/register", {"address": s.address}, api_key=a.admin_key, retries=5)
    elif a.role == "router":
        s = DataRouter(a.host, port, a.admin_key, poll_interval_s=5.0).start()
    else:
        if not a.router:
            ap.error("the gateway needs --router")
        s = DataGateway(a.router, a.host, port, a.admin_key).start()
    print(f"{a.role} listening on {s.address}", flush=True)
    try:
        while not getattr(s, "shutdown_requested", threading.Event()).wait(1.0):
            pass
    except KeyboardInterrupt:
        pass
    s.stop()


if __name__ == "__main__":
    main()
