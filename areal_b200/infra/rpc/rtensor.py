"""Remote tensor handles: batches stay on the worker that produced them; the controller moves
small handles (shard id, node address, layout) and data is fetched over HTTP only when
another worker needs it. Reference: ``areal/infra/rpc/rtensor.py`` and the ``/data`` routes of
``rpc/guard/data_blueprint.py``."""
from __future__ import annotations

import io
import threading
import uuid
from dataclasses import dataclass, field
from typing import Any, Optional

import torch


@dataclass
class TensorShardInfo:
    shard_id: str
    node_addr: str          # host:port of the worker that holds the data
    seqlens: list[int] = field(default_factory=list)   # per-sample token counts (for balancing)
    keys: list[str] = field(default_factory=list)


@dataclass
class RTensor:
    shards: list[TensorShardInfo] = field(default_factory=list)

    @property
    def n_samples(self) -> int:
        return sum(len(s.seqlens) for s in self.shards)

    @property
    def n_tokens(self) -> int:
        return sum(sum(s.seqlens) for s in self.shards)


class ShardStore:
    """Per-process store of batch shards (thread-safe)."""

    def __init__(self):
        self._d: dict[str, Any] = {}
        self._lock = threading.Lock()

    def put(self, batch: dict[str, Any], shard_id: Optional[str] = None) -> str:
        sid = shard_id or uuid.uuid4().hex
        with self._lock:
            self._d[sid] = batch
        return sid

    def get(self, shard_id: str):
        with self._lock:
            if shard_id not in self._d:
                raise KeyError(f"shard {shard_id} not found")
            return self._d[shard_id]

    def delete(self, shard_ids) -> int:
        n = 0
        with self._lock:
            for s in shard_ids:
                n += self._d.pop(s, None) is not None
        return n

    def clear(self):
        with self._lock:
            self._d.clear()

    def __len__(self):
        return len(self._d)


LOCAL_STORE = ShardStore()


def dumps_batch(batch: dict[str, Any]) -> bytes:
    buf = io.BytesIO()
    torch.save(batch, buf)
    return buf.getvalue()


def loads_batch(data: bytes) -> dict[str, Any]:
    return torch.load(io.BytesIO(data), map_location="cpu", weights_only=False)


def remotize(batch: dict[str, Any], node_addr: str, store: ShardStore = LOCAL_STORE) -> RTensor:
    """Stores a padded batch locally and returns its handle."""
    am = batch.get("attention_mask")
    seqlens = am.sum(1).tolist() if am is not None else []
    sid = store.put(batch)
    return RTensor([TensorShardInfo(sid, node_addr, [int(x) for x in seqlens], sorted(k for k in batch))])


def fetch(rt: RTensor, my_addr: Optional[str] = None, store: ShardStore = LOCAL_STORE, timeout: float = 600.0) -> dict[str, Any]:
    """Materialises a handle: local shards come from the store, remote ones over HTTP."""
    import urllib.request

    from ...utils.data import concat_padded_tensors

    parts = []
    for sh in rt.shards:
        if my_addr is not None and sh.node_addr == my_addr:
            parts.append(store.get(sh.shard_id))
        else:
            with urllib.request.urlopen(f"http://{sh.node_addr}/data/{sh.shard_id}", timeout=timeout) as r:
                parts.append(loads_batch(r.read()))
    return concat_padded_tensors(parts) if len(parts) != 1 else parts[0]
