"""Weight-update gateway: pairs a training job with an inference job and drives the transfer.

    POST /connect        {pair, train_workers:[addr], infer_workers:[addr], mode: disk|http, path?}
    POST /update_weights {pair, version}
    POST /disconnect     {pair}
    GET  /weight_meta/{pair}/{key}

``disk``: trainers ``/save`` a Hugging Face checkpoint under ``path/v{version}``, inference
workers load it. ``http``: inference workers pull the weight dictionary that trainer 0 exports
(``GET /weights``, serialised once per version) and hand it to their engine; no shared file system is needed. Generation is paused around the swap and the new version is
published to both sides. Shard-direct GPU transfers (peer-memory push) are driven in-process
by ``areal_b200.parallel.weight_push`` when trainer and rollout ranks share a world.
Reference: ``areal/v2/weight_update/{gateway/app.py, controller.py}``."""
from __future__ import annotations

import os
import threading
import time
from typing import Optional

from ...api.io_struct import SaveLoadMeta
from ...infra.rpc.serialization import serialize_value
from ..common import HTTPError, JsonService, call


class WeightUpdateGateway:
    def __init__(self, host: str = "127.0.0.1", port: Optional[int] = None):
        self.pairs: dict[str, dict] = {}
        self._lock = threading.Lock()
        self.svc = JsonService("weight_update_gateway", host, port)
        self._install()

    def _pair(self, name: str) -> dict:
        with self._lock:
            p = self.pairs.get(name)
        if p is None:
            raise HTTPError(404, f"unknown pair '{name}'")
        return p

    def _install(self):
        svc = self.svc

        @svc.route("GET", "/health")
        def health(body, ctx):
            return {"status": "ok", "pairs": sorted(self.pairs)}

        @svc.route("POST", "/connect")
        def connect(body, ctx):
            mode = body.get("mode", "disk")
            if mode not in ("disk", "http"):
                raise HTTPError(400, f"mode '{mode}' is not served by the gateway (GPU-direct modes run inside the shared world)")
            if mode == "disk" and not body.get("path"):
                raise HTTPError(400, "disk mode needs a shared 'path'")
            p = {"train_workers": list(body["train_workers"]), "infer_workers": list(body["infer_workers"]), "mode": mode,
                 "path": body.get("path"), "version": 0, "history": [], "meta": {}}
            with self._lock:
                self.pairs[body["pair"]] = p
            return {"ok": True, "pair": body["pair"]}

        @svc.route("POST", "/disconnect")
        def disconnect(body, ctx):
            with self._lock:
                self.pairs.pop(body["pair"], None)
            return {"ok": True}

        @svc.route("GET", "/weight_meta/{pair}/{key}")
        def meta(body, ctx):
            p = self._pair(ctx.params["pair"])
            k = ctx.params["key"]
            if k in ("version", "mode", "path"):
                return {k: p[k]}
            if k == "history":
                return {"history": p["history"]}
            if k not in p["meta"]:
                raise HTTPError(404, f"no meta '{k}'")
            return {k: p["meta"][k]}

        @svc.route("POST", "/update_weights")
        def update(body, ctx):
            p = self._pair(body["pair"])
            version = int(body["version"])
            t0 = time.time()
            if p["mode"] == "http":
                for a in p["infer_workers"]:
                    call(f"http://{a}/pause_generation", {})
                try:
                    src = p["train_workers"][0]                # export_weights gathers the whole model on every trainer
                    for a in p["train_workers"]:
                        call(f"http://{a}/set_version", {"version": version})
                    n = [call(f"http://{a}/update_weights_from_http", {"url": f"http://{src}/weights", "version": version})["tensors"]
                         for a in p["infer_workers"]]
                finally:
                    for a in p["infer_workers"]:
                        call(f"http://{a}/continue_generation", {})
                p["version"] = version
                p["history"].append({"version": version, "seconds": time.time() - t0})
                p["meta"]["tensors"] = n[0] if n else 0
                return {"ok": True, "version": version, "seconds": time.time() - t0}
            ckpt = os.path.join(p["path"], f"v{version}")
            for a in p["infer_workers"]:
                call(f"http://{a}/pause_generation", {})
            try:
                meta = SaveLoadMeta(path=ckpt, weight_format="hf", with_optim=False)
                for a in p["train_workers"]:
                    call(f"http://{a}/save", serialize_value({"meta": meta}))
                for a in p["infer_workers"]:
                    call(f"http://{a}/update_weights_from_disk", {"model_path": ckpt, "version": version})
                for a in p["train_workers"]:
                    call(f"http://{a}/set_version", {"version": version})
            finally:
                for a in p["infer_workers"]:
                    call(f"http://{a}/continue_generation", {})
            p["version"] = version
            p["history"].append({"version": version, "seconds": time.time() - t0})
            p["meta"]["last_checkpoint"] = ckpt
            return {"ok": True, "version": version, "seconds": time.time() - t0}

    def start(self):
        self.svc.start()
        return self

    def stop(self):
        self.svc.stop()

    @property
    def address(self) -> str:
        return self.svc.address
