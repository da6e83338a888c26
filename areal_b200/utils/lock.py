"""Distributed lock on a shared filesystem (reference: ``areal/utils/lock.py:10``): atomic
``mkdir`` as the acquire primitive, owner token + stale-lock expiry."""
from __future__ import annotations

import os
import time
import uuid
from typing import Optional


class DistributedLock:
    def __init__(self, name: str, root: str = "/tmp/areal/locks", ttl: float = 600.0):
        self.path = os.path.join(root, name.strip("/").replace("/", "__") + ".lock")
        self.ttl = ttl
        self.token = uuid.uuid4().hex
        os.makedirs(root, exist_ok=True)

    def acquire(self, timeout: Optional[float] = None, poll: float = 0.02) -> bool:
        t0 = time.monotonic()
        while True:
            try:
                os.mkdir(self.path)
                with open(os.path.join(self.path, "owner"), "w") as f:
                    f.write(f"{self.token} {time.time()}")
                return True
            except FileExistsError:
                self._break_if_stale()
            if timeout is not None and time.monotonic() - t0 > timeout:
                return False
            time.sleep(poll)

    def _break_if_stale(self):
        try:
            with open(os.path.join(self.path, "owner")) as f:
                _, ts = f.read().split()
            if time.time() - float(ts) > self.ttl:
                self._remove()
        except (OSError, ValueError):
            pass

    def _remove(self):
        try:
            os.remove(os.path.join(self.path, "owner"))
        except OSError:
            pass
        try:
            os.rmdir(self.path)
        except OSError:
            pass

    def release(self):
        try:
            with open(os.path.join(self.path, "owner")) as f:
                tok = f.read().split()[0]
        except OSError:
            return
        if tok == self.token:
            self._remove()

    def __enter__(self):
        if not self.acquire():
            raise TimeoutError(f"could not acquire {self.path}")
        return self

    def __exit__(self, *exc):
        self.release()
        return False
