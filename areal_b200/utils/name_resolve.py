"""Key-value rendezvous: ``add / get / wait / get_subtree / delete / watch`` with in-memory and
shared-filesystem (NFS) backends and optional TTL keep-alive. Reference:
``areal/utils/name_resolve.py`` (Memory / NFS / Etcd3 / Ray repositories) and ``utils/names.py``.
Etcd and Ray are not available here; selecting them raises a clear error."""
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


# Processes started by a scheduler / launcher inherit the rendezvous location through the
# environment: AREAL_NAME_RESOLVE_ROOT selects the shared-filesystem backend.
_DEFAULT: NameRecordRepository = (NfsNameRecordRepository(os.environ["AREAL_NAME_RESOLVE_ROOT"])
                                  if os.environ.get("AREAL_NAME_RESOLVE_ROOT") else MemoryNameRecordRepository())


def reconfigure(config=None, **kwargs) -> NameRecordRepository:
    """Selects the backend from a ``NameResolveConfig`` (``type``: memory | nfs)."""
    global _DEFAULT
    t = getattr(config, "type", None) or kwargs.get("type", "memory")
    if t == "memory":
        _DEFAULT = MemoryNameRecordRepository()
    elif t == "nfs":
        _DEFAULT = NfsNameRecordRepository(getattr(config, "nfs_record_root", None) or kwargs.get("record_root", "/tmp/areal/name_resolve"))
    elif t in ("etcd3", "ray"):
        raise RuntimeError(f"name_resolve backend '{t}' needs a package that is not installed in this image; use memory or nfs")
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
