"""Key-value rendezvous: ``add / get / wait / get_subtree / delete / watch`` with in-memory and
shared-filesystem (NFS) backends and optional TTL keep-alive. Reference:
``areal/utils/name_resolve.py`` (Memory / NFS / Etcd3 / Ray repositories) and ``utils/names.py``.
The etcd backend speaks etcd's JSON gateway over HTTP (no client package), the Ray backend keeps
the records in a named detached actor."""
from __future__ import annotations

import os
import shutil
import threading
import time
import uuid
from typing import Callable, Optional


class NameEntryExistsError(KeyError):
    pass


class NameEntryNotFoundError(KeyError):
    pass


class NameRecordRepository:
    def add(self, name: str, value: str, delete_on_exit: bool = True, keepalive_ttl: Optional[float] = None,
            replace: bool = False):
        raise NotImplementedError

    def add_subentry(self, name: str, value: str, **kw) -> str:
        sub = f"{name.rstrip('/')}/{uuid.uuid4().hex[:8]}"
        self.add(sub, value, **kw)
        return sub

    def delete(self, name: str):
        raise NotImplementedError

    def clear_subtree(self, name_root: str):
        raise NotImplementedError

    def get(self, name: str) -> str:
        raise NotImplementedError

    def get_subtree(self, name_root: str) -> list[str]:
        raise NotImplementedError

    def find_subtree(self, name_root: str) -> list[str]:
        raise NotImplementedError

    def wait(self, name: str, timeout: Optional[float] = None, poll_frequency: float = 0.1) -> str:
        t0 = time.monotonic()
        while True:
            try:
                return self.get(name)
            except NameEntryNotFoundError:
                if timeout is not None and time.monotonic() - t0 > timeout:
                    raise TimeoutError(f"timed out waiting for key '{name}'")
                time.sleep(poll_frequency)

    def watch_names(self, names, call_back: Callable[[], None], poll_frequency: float = 1.0, wait_timeout: float = 300):
        """Calls ``call_back`` once any of ``names`` disappears (e.g. a worker died)."""
        names = [names] if isinstance(names, str) else list(names)

        def run():
            for n in names:
                try:
                    self.wait(n, timeout=wait_timeout, poll_frequency=poll_frequency)
                except TimeoutError:
                    return
            while True:
                for n in names:
                    try:
                        self.get(n)
                    except NameEntryNotFoundError:
                        call_back()
                        return
                time.sleep(poll_frequency)

        t = threading.Thread(target=run, daemon=True)
        t.start()
        return t

    def reset(self):
        pass


class MemoryNameRecordRepository(NameRecordRepository):
    _store: dict[str, str] = {}
    _lock = threading.Lock()

    def __init__(self):
        self._mine: set[str] = set()

    def add(self, name, value, delete_on_exit=True, keepalive_ttl=None, replace=False):
        name = name.rstrip("/")
        with self._lock:
            if name in self._store and not replace:
                raise NameEntryExistsError(name)
            self._store[name] = str(value)
        if delete_on_exit:
            self._mine.add(name)

    def delete(self, name):
        with self._lock:
            if name not in self._store:
                raise NameEntryNotFoundError(name)
            del self._store[name]
        self._mine.discard(name)

    def clear_subtree(self, name_root):
        with self._lock:
            for k in [k for k in self._store if k.startswith(name_root.rstrip("/"))]:
                del self._store[k]

    def get(self, name):
        with self._lock:
            if name.rstrip("/") not in self._store:
                raise NameEntryNotFoundError(name)
            return self._store[name.rstrip("/")]

    def get_subtree(self, name_root):
        with self._lock:
            return [v for k, v in sorted(self._store.items()) if k.startswith(name_root.rstrip("/"))]

    def find_subtree(self, name_root):
        with self._lock:
            return sorted(k for k in self._store if k.startswith(name_root.rstrip("/")))

    def reset(self):
        for n in list(self._mine):
            try:
                self.delete(n)
            except NameEntryNotFoundError:
                pass


class NfsNameRecordRepository(NameRecordRepository):
    """One file per key under ``record_root`` (works across processes and nodes that share it)."""

    def __init__(self, record_root: str = "/tmp/areal/name_resolve"):
        self.root = record_root
        self._mine: set[str] = set()
        os.makedirs(self.root, exist_ok=True)

    def _path(self, name: str) -> str:
        return os.path.join(self.root, name.strip("/"), "ENTRY")

    def add(self, name, value, delete_on_exit=True, keepalive_ttl=None, replace=False):
        p = self._path(name)
        if os.path.isfile(p) and not replace:
            raise NameEntryExistsError(name)
        os.makedirs(os.path.dirname(p), exist_ok=True)
        tmp = p + f".tmp{uuid.uuid4().hex[:6]}"
        with open(tmp, "w") as f:
            f.write(str(value))
        os.replace(tmp, p)
        if delete_on_exit:
            self._mine.add(name)

    def delete(self, name):
        p = self._path(name)
        if not os.path.isfile(p):
            raise NameEntryNotFoundError(name)
        os.remove(p)
        self._mine.discard(name)
        d = os.path.dirname(p)
        while d != self.root and os.path.isdir(d) and not os.listdir(d):
            os.rmdir(d)
            d = os.path.dirname(d)

    def clear_subtree(self, name_root):
        shutil.rmtree(os.path.join(self.root, name_root.strip("/")), ignore_errors=True)

    def get(self, name):
        p = self._path(name)
        for _ in range(3):  # tolerate NFS attribute-cache lag
            try:
                with open(p) as f:
                    return f.read()
            except FileNotFoundError:
                time.sleep(0.01)
        raise NameEntryNotFoundError(name)

    def find_subtree(self, name_root):
        base = os.path.join(self.root, name_root.strip("/"))
        out = []
        for d, _, files in os.walk(base):
            if "ENTRY" in files:
                out.append(os.path.relpath(d, self.root))
        return sorted(out)

    def get_subtree(self, name_root):
        return [self.get(k) for k in self.find_subtree(name_root)]

    def reset(self):
        for n in list(self._mine):
            try:
                self.delete(n)
            except NameEntryNotFoundError:
                pass


class Etcd3NameRecordRepository(NameRecordRepository):
    """Records in an etcd v3 cluster, spoken to through etcd's own JSON gateway (``/v3/kv/put``,
    ``/v3/kv/range``, ``/v3/kv/deleterange``, ``/v3/lease/grant``, ``/v3/lease/keepalive``): no
    client package is needed. ``keepalive_ttl`` attaches a lease that a background thread renews
    until the entry is deleted, so entries of a process that died disappear on their own
    (reference: ``areal/utils/name_resolve.py:414`` Etcd3NameRecordRepository)."""

    def __init__(self, addr: str = "localhost:2379", timeout: float = 5.0):
        import base64
        import json as _json
        import urllib.request

        self._b64 = lambda s_: base64.b64encode(s_.encode()).decode()
        self._unb64 = lambda s_: base64.b64decode(s_).decode()
        self._json, self._req = _json, urllib.request
        self.base = addr if addr.startswith("http") else f"http://{addr}"
        self.timeout = timeout
        self._mine: set[str] = set()
        self._leases: dict[str, tuple[str, float, float]] = {}    # name -> (lease id, ttl, next renewal)
        self._lock = threading.Lock()
        self._stop = threading.Event()
        self._keeper: Optional[threading.Thread] = None

    def _call(self, path: str, body: dict) -> dict:
        req = self._req.Request(self.base + path, data=self._json.dumps(body).encode(), headers={"Content-Type": "application/json"})
        with self._req.urlopen(req, timeout=self.timeout) as r:
            return self._json.loads(r.read().decode() or "{}")

    @staticmethod
    def _range_end(prefix: str) -> str:
        b = bytearray(prefix.encode())
        b[-1] += 1
        return bytes(b).decode("latin-1")

    def _keepalive_loop(self):
        while not self._stop.wait(0.2):
            now = time.monotonic()
            with self._lock:
                due = [(n, lid, ttl) for n, (lid, ttl, nxt) in self._leases.items() if now >= nxt]
            for n, lid, ttl in due:
                try:
                    self._call("/v3/lease/keepalive", {"ID": lid})
                except Exception:
                    pass
                with self._lock:
                    if n in self._leases:
                        self._leases[n] = (lid, ttl, now + max(0.2, ttl / 3))

    def add(self, name, value, delete_on_exit=True, keepalive_ttl=None, replace=False):
        name = name.rstrip("/")
        if not replace:
            try:
                self.get(name)
                raise NameEntryExistsError(name)
            except NameEntryNotFoundError:
                pass
        body = {"key": self._b64(name), "value": self._b64(str(value))}
        if keepalive_ttl:
            lease = self._call("/v3/lease/grant", {"TTL": int(max(1, keepalive_ttl))})
            body["lease"] = lease["ID"]
            with self._lock:
                self._leases[name] = (lease["ID"], float(keepalive_ttl), time.monotonic() + keepalive_ttl / 3)
            if self._keeper is None:
                self._keeper = threading.Thread(target=self._keepalive_loop, name="etcd-keepalive", daemon=True)
                self._keeper.start()
        self._call("/v3/kv/put", body)
        if delete_on_exit:
            self._mine.add(name)
        return name

    def delete(self, name):
        name = name.rstrip("/")
        res = self._call("/v3/kv/deleterange", {"key": self._b64(name)})
        with self._lock:
            self._leases.pop(name, None)
        self._mine.discard(name)
        if int(res.get("deleted", 0) or 0) == 0:
            raise NameEntryNotFoundError(name)

    def clear_subtree(self, name_root):
        root = name_root.rstrip("/") + "/"
        self._call("/v3/kv/deleterange", {"key": self._b64(root), "range_end": self._b64(self._range_end(root))})
        try:
            self._call("/v3/kv/deleterange", {"key": self._b64(name_root.rstrip("/"))})
        except Exception:
            pass

    def get(self, name):
        res = self._call("/v3/kv/range", {"key": self._b64(name.rstrip("/"))})
        kvs = res.get("kvs") or []
        if not kvs:
            raise NameEntryNotFoundError(name)
        return self._unb64(kvs[0]["value"])

    def _range(self, name_root):
        root = name_root.rstrip("/") + "/"
        res = self._call("/v3/kv/range", {"key": self._b64(root), "range_end": self._b64(self._range_end(root))})
        return sorted((self._unb64(kv["key"]), self._unb64(kv["value"])) for kv in (res.get("kvs") or []))

    def get_subtree(self, name_root):
        return [v for _, v in self._range(name_root)]

    def find_subtree(self, name_root):
        return [k for k, _ in self._range(name_root)]

    def reset(self):
        self._stop.set()
        for n in list(self._mine):
            try:
                self.delete(n)
            except Exception:
                pass


class RayNameRecordRepository(NameRecordRepository):
    """Records in a named, detached Ray actor that every process of the job can look up (reference:
    ``areal/utils/name_resolve.py:885`` RayNameResolveRepository). ``ray_module`` lets tests hand in a
    stand-in for the ``ray`` package."""

    class _Store:
        def __init__(self):
            self.kv: dict[str, str] = {}

        def put(self, k, v, replace):
            if k in self.kv and not replace:
                return False
            self.kv[k] = v
            return True

        def get(self, k):
            return self.kv.get(k)

        def delete(self, k):
            return self.kv.pop(k, None) is not None

        def prefix(self, root):
            return sorted((k, v) for k, v in self.kv.items() if k.startswith(root))

        def clear(self, root):
            for k in [k for k in self.kv if k == root.rstrip("/") or k.startswith(root)]:
                del self.kv[k]

    def __init__(self, actor_name: str = "ray_kv_store", ray_module=None):
        if ray_module is None:
            import ray as ray_module  # noqa: F811  (only needed for this backend)
        self.ray = ray_module
        if not self.ray.is_initialized():
            self.ray.init(ignore_reinit_error=True)
        try:
            self.actor = self.ray.get_actor(actor_name)
        except Exception:
            self.actor = self.ray.remote(self._Store).options(name=actor_name, lifetime="detached", get_if_exists=True).remote()
        self._mine: set[str] = set()

    def _do(self, method: str, *a):
        return self.ray.get(getattr(self.actor, method).remote(*a))

    def add(self, name, value, delete_on_exit=True, keepalive_ttl=None, replace=False):
        name = name.rstrip("/")
        if not self._do("put", name, str(value), bool(replace)):
            raise NameEntryExistsError(name)
        if delete_on_exit:
            self._mine.add(name)
        return name

    def delete(self, name):
        name = name.rstrip("/")
        self._mine.discard(name)
        if not self._do("delete", name):
            raise NameEntryNotFoundError(name)

    def clear_subtree(self, name_root):
        self._do("clear", name_root.rstrip("/") + "/")

    def get(self, name):
        v = self._do("get", name.rstrip("/"))
        if v is None:
            raise NameEntryNotFoundError(name)
        return v

    def get_subtree(self, name_root):
        return [v for _, v in self._do("prefix", name_root.rstrip("/") + "/")]

    def find_subtree(self, name_root):
        return [k for k, _ in self._do("prefix", name_root.rstrip("/") + "/")]

    def reset(self):
        for n in list(self._mine):
            try:
                self.delete(n)
            except Exception:
                pass


# Processes started by a scheduler / launcher inherit the rendezvous location through the
# environment: AREAL_NAME_RESOLVE_ROOT selects the shared-filesystem backend.
_DEFAULT: NameRecordRepository = (NfsNameRecordRepository(os.environ["AREAL_NAME_RESOLVE_ROOT"])
                                  if os.environ.get("AREAL_NAME_RESOLVE_ROOT") else MemoryNameRecordRepository())


def reconfigure(config=None, **kwargs) -> NameRecordRepository:
    """Selects the backend from a ``NameResolveConfig`` (``type``: memory | nfs | etcd3 | ray)."""
    global _DEFAULT
    t = getattr(config, "type", None) or kwargs.get("type", "memory")
    if t == "memory":
        _DEFAULT = MemoryNameRecordRepository()
    elif t == "nfs":
        _DEFAULT = NfsNameRecordRepository(getattr(config, "nfs_record_root", None) or kwargs.get("record_root", "/tmp/areal/name_resolve"))
    elif t == "etcd3":
        _DEFAULT = Etcd3NameRecordRepository(getattr(config, "etcd3_addr", None) or kwargs.get("addr", "localhost:2379"))
    elif t == "ray":
        _DEFAULT = RayNameRecordRepository(getattr(config, "ray_actor_name", None) or kwargs.get("actor_name", "ray_kv_store"),
                                           ray_module=kwargs.get("ray_module"))
    else:
        raise ValueError(f"unknown name_resolve backend '{t}'")
    return _DEFAULT


def add(*a, **k): return _DEFAULT.add(*a, **k)
def add_subentry(*a, **k): return _DEFAULT.add_subentry(*a, **k)
def delete(*a, **k): return _DEFAULT.delete(*a, **k)
def clear_subtree(*a, **k): return _DEFAULT.clear_subtree(*a, **k)
def get(*a, **k): return _DEFAULT.get(*a, **k)
def get_subtree(*a, **k): return _DEFAULT.get_subtree(*a, **k)
def find_subtree(*a, **k): return _DEFAULT.find_subtree(*a, **k)
def wait(*a, **k): return _DEFAULT.wait(*a, **k)
def watch_names(*a, **k): return _DEFAULT.watch_names(*a, **k)
def reset(): return _DEFAULT.reset()
