"""Training service front: a registry of workers with their place in the parallel layout (router) and one keyed entry
point that dispatches batches by that topology (gateway).

A worker announces ``{address, rank, dp_rank, dp_size, is_dp_head}`` (``TrainingWorker.topology()`` reads it from its
engine). Data-parallel groups get different shares of a batch, split by token count; the model-parallel peers of a group
(tensor / pipeline / sequence-parallel ranks that must see the same rows) get the SAME share as their head, at the same
time, so their collectives line up; answers are taken from the heads and merged back into the caller's order. Calls
that carry no batch (save, load, set_version, step_lr_scheduler) go to every worker.

Routes of the gateway (``Authorization: Bearer <admin key>`` when a key is set):
    GET  /health              GET /topology
    POST /call                {"route": "/ppo/actor/update", "batch": <envelope>, "kwargs": {...}}  -> {"result": <envelope>}
    POST /broadcast           {"route": "/set_version", "body": {...}}
Routes of the router:
    POST /register | /unregister | /heartbeat        GET /workers | /health

Reference: ``areal/v2/training_service/{router/{app,state}.py, gateway/engine.py, data_proxy/{dispatcher,topology}.py}``.
"""
from __future__ import annotations

import concurrent.futures as cf
import threading
import time
from typing import Any, Optional

from ...infra.controller.train_controller import merge_results, split_batch
from ...infra.rpc.serialization import deserialize_value, serialize_value
from ..common import HTTPError, JsonService, call


class TrainingRouter:
    """Worker registry: who is there, where each sits in the layout, who stopped answering."""

    def __init__(self, host: str = "127.0.0.1", port: Optional[int] = None, heartbeat_timeout: float = 30.0):
        self.workers: dict[str, dict] = {}
        self.heartbeat_timeout = heartbeat_timeout
        self._lock = threading.Lock()
        self.svc = JsonService("training_router", host, port)
        self._install()

    def live(self) -> list[dict]:
        now = time.monotonic()
        with self._lock:
            return [dict(w, address=a) for a, w in sorted(self.workers.items(), key=lambda kv: kv[1]["rank"])
                    if now - w["seen"] <= self.heartbeat_timeout]

    def groups(self) -> list[list[dict]]:
        """Live workers by data-parallel rank, the head of each group first. Raises 503 while a group is incomplete."""
        live = self.live()
        if not live:
            raise HTTPError(503, "no training worker registered")
        dp = max(w["dp_size"] for w in live)
        out: list[list[dict]] = [[] for _ in range(dp)]
        for w in live:
            out[w["dp_rank"]].append(w)
        per = {len(g) for g in out}
        if len(per) != 1 or 0 in per or sum(1 for g in out for w in g if w["is_dp_head"]) != dp:
            raise HTTPError(503, f"training workers incomplete: data-parallel groups of sizes {[len(g) for g in out]}")
        return [sorted(g, key=lambda w: (not w["is_dp_head"], w["rank"])) for g in out]

    def _install(self):
        svc = self.svc

        @svc.route("POST", "/register")
        def register(body, ctx):
            w = {k: body[k] for k in ("rank", "dp_rank", "dp_size", "is_dp_head")}
            w["seen"] = time.monotonic()
            with self._lock:
                self.workers[body["address"]] = w
            return {"ok": True, "workers": len(self.workers)}

        @svc.route("POST", "/unregister")
        def unregister(body, ctx):
            with self._lock:
                self.workers.pop(body["address"], None)
            return {"ok": True}

        @svc.route("POST", "/heartbeat")
        def heartbeat(body, ctx):
            with self._lock:
                w = self.workers.get(body["address"])
                if w is None:
                    raise HTTPError(404, "unknown worker: register first")
                w["seen"] = time.monotonic()
            return {"ok": True}

        @svc.route("GET", "/workers")
        def workers(body, ctx):
            return {"workers": self.live()}

        @svc.route("GET", "/health")
        def health(body, ctx):
            return {"status": "ok", "registered": len(self.workers), "live": len(self.live())}

    def start(self):
        self.svc.start()
        return self

    def stop(self):
        self.svc.stop()


class TrainingGateway:
    def __init__(self, router: TrainingRouter, host: str = "127.0.0.1", port: Optional[int] = None, admin_key: Optional[str] = None,
                 group_size: int = 1, timeout: float = 7200.0):
        self.router, self.admin_key, self.group_size, self.timeout = router, admin_key, group_size, timeout
        self._pool = cf.ThreadPoolExecutor(max_workers=64)
        self.svc = JsonService("training_gateway", host, port)
        self._install()

    def _auth(self, ctx):
        if self.admin_key and ctx.api_key != self.admin_key:
            raise HTTPError(401, "bad admin key")

    def dispatch(self, route: str, batch: dict[str, Any], kwargs: Optional[dict] = None):
        groups = self.router.groups()
        n = len(groups)
        B = batch["attention_mask"].shape[0]
        subs, idx = split_batch(batch, n, self.group_size) if n > 1 else ([batch], [list(range(B))])
        futs = []
        for g, sub in zip(groups, subs):
            body = serialize_value({"batch": sub, **(kwargs or {})})            # serialised once per group, sent to all its ranks
            futs.append([self._pool.submit(call, f"http://{w['address']}{route}", body, None, None, self.timeout) for w in g])
        outs = []
        for fs in futs:
            res = [f.result() for f in fs]                                        # every rank must finish; the head's answer counts
            outs.append(deserialize_value(res[0]["result"]))
        return merge_results(outs, idx, seq_len=batch["attention_mask"].shape[1])

    def broadcast(self, route: str, body: Optional[dict] = None, method: str = "POST") -> list[dict]:
        ws = [w for g in self.router.groups() for w in g]
        futs = [self._pool.submit(call, f"http://{w['address']}{route}", body if method == "POST" else None, method, None, self.timeout) for w in ws]
        return [f.result() for f in futs]

    def _install(self):
        svc = self.svc

        @svc.route("GET", "/health")
        def health(body, ctx):
            try:
                g = self.router.groups()
                return {"status": "ok", "dp_size": len(g), "workers": sum(len(x) for x in g)}
            except HTTPError as e:
                return 503, {"status": "degraded", "error": e.message}

        @svc.route("GET", "/topology")
        def topology(body, ctx):
            self._auth(ctx)
            return {"groups": [[{k: w[k] for k in ("address", "rank", "dp_rank", "is_dp_head")} for w in g] for g in self.router.groups()]}

        @svc.route("POST", "/call")
        def call_(body, ctx):
            self._auth(ctx)
            args = deserialize_value(body)
            res = self.dispatch(args["route"], args["batch"], args.get("kwargs"))
            return {"result": serialize_value(res)}

        @svc.route("POST", "/broadcast")
        def bcast(body, ctx):
            self._auth(ctx)
            return {"results": self.broadcast(body["route"], body.get("body") or {}, body.get("method", "POST"))}

    def start(self):
        self.svc.start()
        return self

    def stop(self):
        self.svc.stop()
        self._pool.shutdown(wait=False)


class GatewayTrainingClient:
    """The caller's side of the gateway: the method names of a train engine, one address, one key."""

    def __init__(self, gateway_address: str, admin_key: Optional[str] = None, timeout: float = 7200.0):
        self.url, self.key, self.timeout = f"http://{gateway_address}", admin_key, timeout
        self._version = 0

    def _call(self, route: str, batch: dict, **kwargs):
        r = call(f"{self.url}/call", serialize_value({"route": route, "batch": batch, "kwargs": kwargs}), api_key=self.key, timeout=self.timeout)
        res = deserialize_value(r["result"])
        if isinstance(res, dict) and "attention_mask" in res:
            batch.update(res)
            return batch
        return res

    def _all(self, route: str, body: Optional[dict] = None, method: str = "POST"):
        return call(f"{self.url}/broadcast", {"route": route, "body": body or {}, "method": method}, api_key=self.key, timeout=self.timeout)["results"]

    def compute_logp(self, batch):
        return self._call("/ppo/actor/compute_logp", batch)

    def compute_advantages(self, batch, **kw):
        return self._call("/ppo/actor/compute_advantages", batch, **kw)

    def ppo_update(self, batch):
        return self._call("/ppo/actor/update", batch)

    def compute_values(self, batch):
        return self._call("/ppo/critic/compute_values", batch)

    def train_lm(self, batch):
        return self._call("/sft/train", batch)

    def train_rw(self, batch):
        return self._call("/rw/train", batch)

    def train_dpo(self, batch):
        return self._call("/dpo/train", batch)

    def forward_batch(self, batch, **kw):
        return self._call("/forward", batch, **kw)

    def set_version(self, version: int):
        self._version = int(version)
        self._all("/set_version", {"version": int(version)})

    def get_version(self) -> int:
        return self._version

    def step_lr_scheduler(self):
        self._all("/step_lr_scheduler")

    def save(self, meta):
        self._all("/save", serialize_value({"meta": meta}))

    def load(self, meta):
        self._all("/load", serialize_value({"meta": meta}))

    def topology(self) -> list[list[dict]]:
        return call(f"{self.url}/topology", api_key=self.key)["groups"]
