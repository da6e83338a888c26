"""Trainer-side stub of the rollout controller: an object with the slice of the
``InferenceEngine`` API a train engine needs (pause / resume / versions / weight sync /
rollout_batch) that forwards each call to the controller's callback server. Reference:
``areal/infra/controller/rollout_callback.py``."""
from __future__ import annotations

from typing import Any, Optional

from ...api.io_struct import WeightUpdateMeta
from ..scheduler.local import http_json
from ..rpc.serialization import deserialize_value


class RolloutCallback:
    def __init__(self, controller_addr: str, timeout: float = 3600.0):
        self.addr = controller_addr
        self.timeout = timeout

    def _call(self, name: str, *args, **kwargs) -> Any:
        r = http_json(f"http://{self.addr}/callback/{name}", {"args": list(args), "kwargs": kwargs}, timeout=self.timeout)
        if "__http_error__" in r or "error" in r:
            raise RuntimeError(f"rollout callback '{name}' failed: {r.get('error')}")
        return deserialize_value(r.get("result"))

    def pause(self):
        return self._call("pause")

    def resume(self):
        return self._call("resume")

    def pause_generation(self):
        return self._call("pause_generation")

    def continue_generation(self):
        return self._call("continue_generation")

    def set_version(self, version: int):
        return self._call("set_version", version)

    def get_version(self) -> int:
        return int(self._call("get_version"))

    def update_weights_from_disk(self, meta: WeightUpdateMeta):
        return self._call("update_weights_from_disk", meta)

    def update_weights_from_handle(self, handle, meta: Optional[WeightUpdateMeta] = None):
        return self._call("update_weights_from_handle", handle, meta)

    def rollout_batch(self, data, workflow: Optional[str] = None, workflow_kwargs: Optional[dict] = None,
                      should_accept_fn: Optional[str] = None):
        return self._call("rollout_batch", data, workflow=workflow, workflow_kwargs=workflow_kwargs,
                          should_accept_fn=should_accept_fn)

    def export_stats(self) -> dict:
        return self._call("export_stats")
