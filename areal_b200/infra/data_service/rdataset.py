"""Remote datasets: a ``DatasetWorker`` process hosts a dataset behind HTTP (length, item
fetch by index list); ``RDataset`` is the ``torch.utils.data.Dataset`` client with a prefetch
buffer that fetches the sampler's upcoming indices in batches on a background thread, so a
controller process can iterate data that lives next to storage. Reference:
``areal/infra/data_service/*`` (``rdataset.py:36-330`` RDataset + prefetch-aware sampler)."""
from __future__ import annotations

import collections
import threading
from typing import Any, Iterable, Optional, Sequence

from torch.utils.data import Dataset, Sampler

from ...v2.common import HTTPError, JsonService, call
from ..rpc.serialization import deserialize_value, serialize_value


class DatasetWorker:
    def __init__(self, dataset, host: str = "127.0.0.1", port: Optional[int] = None, name: str = "default"):
        self.dataset, self.name = dataset, name
        self.svc = JsonService("dataset_worker", host, port)

        @self.svc.route("GET", "/health")
        def health(body, ctx):
            return {"status": "ok", "name": self.name, "len": len(self.dataset)}

        @self.svc.route("GET", "/len")
        def length(body, ctx):
            return {"len": len(self.dataset)}

        @self.svc.route("POST", "/items")
        def items(body, ctx):
            idx = body["indices"]
            n = len(self.dataset)
            if any(i < 0 or i >= n for i in idx):
                raise HTTPError(400, "index out of range")
            return {"items": [serialize_value(self.dataset[i]) for i in idx]}

    def start(self):
        self.svc.start()
        return self

    def stop(self):
        self.svc.stop()

    @property
    def address(self) -> str:
        return self.svc.address


class RDataset(Dataset):
    def __init__(self, address: str, prefetch: int = 64, timeout: float = 60.0, token: Optional[str] = None,
                 length: Optional[int] = None, dataset_id: Optional[str] = None):
        """``address``: a :class:`DatasetWorker` (no token) or the gateway of the data service (``token``: the key the
        gateway handed out when the dataset was registered)."""
        self.address, self.timeout = address, timeout
        self.token, self.dataset_id = token, dataset_id
        self._len = int(length) if length is not None else int(call(f"http://{address}/len", timeout=timeout)["len"])
        self.prefetch = prefetch
        self._cache: "collections.OrderedDict[int, Any]" = collections.OrderedDict()
        self._lock = threading.Lock()
        self._pending: set[int] = set()
        self._cv = threading.Condition(self._lock)

    def __len__(self) -> int:
        return self._len

    def _fetch(self, indices: Sequence[int]) -> None:
        try:
            if self.token is not None:
                items = call(f"http://{self.address}/v1/samples/fetch", {"indices": list(indices)}, api_key=self.token,
                             timeout=self.timeout)["samples"]
            else:
                items = call(f"http://{self.address}/items", {"indices": list(indices)}, timeout=self.timeout)["items"]
            with self._cv:
                for i, it in zip(indices, items):
                    self._cache[i] = deserialize_value(it)
                    self._pending.discard(i)
                while len(self._cache) > 4 * max(1, self.prefetch):
                    self._cache.popitem(last=False)
                self._cv.notify_all()
        except BaseException:
            with self._cv:
                for i in indices:
                    self._pending.discard(i)
                self._cv.notify_all()
            raise

    def advance_epoch(self, epoch: Optional[int] = None) -> int:
        """Tells the service that a new epoch starts (datasets that reshuffle or re-augment per epoch follow)."""
        if self.token is None:
            return 0
        body = {} if epoch is None else {"epoch": int(epoch)}
        return int(call(f"http://{self.address}/v1/epochs/advance", body, api_key=self.token, timeout=self.timeout)["epoch"])

    def save_state(self, path: str) -> list:
        return call(f"http://{self.address}/v1/state/save", {"path": path}, api_key=self.token, timeout=self.timeout)["files"]

    def load_state(self, path: str) -> dict:
        return call(f"http://{self.address}/v1/state/load", {"path": path}, api_key=self.token, timeout=self.timeout)

    def hint(self, upcoming: Iterable[int]) -> None:
        """Announces indices that will be requested soon; they are fetched in the background."""
        with self._lock:
            need = [i for i in upcoming if i not in self._cache and i not in self._pending][: self.prefetch]
            self._pending.update(need)
        if need:
            threading.Thread(target=self._fetch, args=(need,), daemon=True).start()

    def __getitem__(self, i: int):
        if i < 0 or i >= self._len:
            raise IndexError(i)
        with self._cv:
            while i in self._pending:
                self._cv.wait(timeout=self.timeout)
            if i in self._cache:
                return self._cache.pop(i)
        self._fetch([i])
        with self._lock:
            return self._cache.pop(i)


class PrefetchAwareSampler(Sampler):
    """Wraps a sampler and tells the :class:`RDataset` which indices come next."""

    def __init__(self, base: Sampler, dataset: RDataset, lookahead: int = 64):
        self.base, self.dataset, self.lookahead = base, dataset, lookahead

    def __len__(self):
        return len(self.base)

    def __iter__(self):
        order = list(iter(self.base))
        for k, i in enumerate(order):
            if k % max(1, self.lookahead // 2) == 0:
                self.dataset.hint(order[k:k + self.lookahead])
            yield i
