"""Process helpers: kill a whole process tree / group by exact pid (never by name).
Reference: ``areal/infra/utils/proc.py``."""
from __future__ import annotations

import os
import signal
import subprocess
import time
from typing import Optional


def kill_process_tree(pid: int, sig: int = signal.SIGTERM, grace: float = 5.0, include_parent: bool = True) -> None:
    try:
        import psutil
    except ImportError:  # pragma: no cover
        psutil = None
    if psutil is None:
        try:
            os.kill(pid, sig)
        except ProcessLookupError:
            pass
        return
    try:
        parent = psutil.Process(pid)
    except psutil.NoSuchProcess:
        return
    procs = parent.children(recursive=True) + ([parent] if include_parent else [])
    for p in procs:
        try:
            p.send_signal(sig)
        except psutil.NoSuchProcess:
            pass
    _, alive = psutil.wait_procs(procs, timeout=grace)
    for p in alive:
        try:
            p.kill()
        except psutil.NoSuchProcess:
            pass


def terminate_popen(p: subprocess.Popen, grace: float = 10.0) -> Optional[int]:
    """Stops a child started with ``start_new_session=True`` together with its group."""
    if p.poll() is not None:
        return p.returncode
    try:
        os.killpg(os.getpgid(p.pid), signal.SIGTERM)
    except (ProcessLookupError, PermissionError):
        p.terminate()
    t0 = time.monotonic()
    while p.poll() is None and time.monotonic() - t0 < grace:
        time.sleep(0.05)
    if p.poll() is None:
        try:
            os.killpg(os.getpgid(p.pid), signal.SIGKILL)
        except (ProcessLookupError, PermissionError):
            p.kill()
        p.wait(timeout=5)
    return p.returncode
