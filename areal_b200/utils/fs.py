"""Filesystem helpers for shared storage (reference: ``areal/utils/fs.py``)."""
from __future__ import annotations

import getpass
import os
import shutil
import tempfile
import time


def get_user_tmp() -> str:
    d = os.path.join(tempfile.gettempdir(), f"areal-{getpass.getuser()}")
    os.makedirs(d, exist_ok=True)
    return d


def atomic_write(path: str, data, mode: str = "w") -> None:
    """Write-then-rename so readers on a shared filesystem never see a torn file."""
    os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    tmp = f"{path}.tmp{os.getpid()}"
    with open(tmp, mode) as f:
        f.write(data)
        f.flush()
        os.fsync(f.fileno())
    os.replace(tmp, path)


def wait_for_path(path: str, timeout: float = 60.0, poll: float = 0.2) -> bool:
    """NFS-safe wait: listing the parent directory refreshes the attribute cache."""
    t0 = time.monotonic()
    while time.monotonic() - t0 < timeout:
        try:
            os.listdir(os.path.dirname(os.path.abspath(path)))
        except OSError:
            pass
        if os.path.exists(path):
            return True
        time.sleep(poll)
    return False


def remove_tree(path: str, retries: int = 3) -> None:
    for i in range(retries):
        try:
            shutil.rmtree(path)
            return
        except FileNotFoundError:
            return
        except OSError:
            time.sleep(0.2 * (i + 1))
    shutil.rmtree(path, ignore_errors=True)


def dir_size_bytes(path: str) -> int:
    tot = 0
    for root, _, files in os.walk(path):
        for f in files:
            try:
                tot += os.path.getsize(os.path.join(root, f))
            except OSError:
                pass
    return tot
