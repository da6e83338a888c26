"""Inference-service controller: brings up router, gateway and one data proxy per engine in
this process (or registers remote proxies), and offers the ``InferenceEngine``-shaped surface
a trainer needs on top of the HTTP API: run agents against the gateway, collect exported
trajectories as training batches, pause / resume, publish versions. Reference:
``areal/v2/inference_service/controller/controller.py``."""
from __future__ import annotations

from typing import Any, Callable, Optional

import torch

from ...utils.data import concat_padded_tensors
from ..common import call
from .data_proxy import DataProxy
from .gateway import Gateway
from .router import Router


class InferenceServiceController:
    def __init__(self, admin_key: str = "areal-admin-key"):
        self.admin_key = admin_key
        self.router: Optional[Router] = None
        self.gateway: Optional[Gateway] = None
        self.proxies: list[DataProxy] = []
        self._version = 0

    def start(self, engines: list, tokenizer, gconfig=None, chat_template_type: str = "hf"):
        self.router = Router().start()
        for e in engines:
            p = DataProxy(e, tokenizer, gconfig, chat_template_type=chat_template_type).start()
            self.proxies.append(p)
            call(f"http://{self.router.address}/register", {"address": p.address})
        self.gateway = Gateway(self.router.address, self.admin_key).start()
        return self

    def register_remote_proxy(self, address: str):
        call(f"http://{self.router.address}/register", {"address": address})

    @property
    def base_url(self) -> str:
        return f"{self.gateway.svc.url}/v1"

    # ---- sessions
    def start_session(self, task_id: Optional[str] = None) -> dict:
        return call(f"{self.gateway.svc.url}/rl/start_session", {"task_id": task_id}, api_key=self.admin_key)

    def export_batch(self, style: str = "individual", discount: float = 1.0) -> Optional[dict[str, Any]]:
        """Finished sessions' trajectories as one padded training batch."""
        r = call(f"{self.gateway.svc.url}/export_trajectories", {"style": style, "discount": discount}, api_key=self.admin_key)
        trajs = []
        for s in r["sessions"]:
            for t in s["trajectories"]:
                trajs.append({
                    "input_ids": torch.tensor(t["input_ids"], dtype=torch.long).unsqueeze(0),
                    "loss_mask": torch.tensor(t["loss_mask"], dtype=torch.int32).unsqueeze(0),
                    "logprobs": torch.tensor(t["logprobs"], dtype=torch.float32).unsqueeze(0),
                    "versions": torch.tensor(t["versions"], dtype=torch.int32).unsqueeze(0),
                    "attention_mask": torch.ones(1, len(t["input_ids"]), dtype=torch.bool),
                    "rewards": torch.tensor(t["rewards"], dtype=torch.float32),
                })
        return concat_padded_tensors(trajs) if trajs else None

    # ---- control plane
    def _admin(self, path: str, body: Optional[dict] = None):
        return call(f"{self.gateway.svc.url}{path}", body or {}, api_key=self.admin_key)

    def pause_generation(self):
        self._admin("/pause_generation")

    def continue_generation(self):
        self._admin("/continue_generation")

    def set_version(self, version: int):
        self._version = version
        self._admin("/set_version", {"version": version})

    def get_version(self) -> int:
        return self._version

    def stop(self):
        if self.gateway:
            self.gateway.stop()
        for p in self.proxies:
            p.stop()
        if self.router:
            self.router.stop()
