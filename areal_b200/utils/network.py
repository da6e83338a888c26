"""Host / port helpers (reference: ``areal/utils/network.py``)."""
from __future__ import annotations

import random
import socket
from contextlib import closing


def gethostname() -> str:
    return socket.gethostname()


def gethostip() -> str:
    try:
        with closing(socket.socket(socket.AF_INET, socket.SOCK_DGRAM)) as s:
            s.connect(("10.255.255.255", 1))
            return s.getsockname()[0]
    except OSError:
        return "127.0.0.1"


def is_port_free(port: int, host: str = "") -> bool:
    with closing(socket.socket(socket.AF_INET, socket.SOCK_STREAM)) as s:
        s.setsockopt(socket.SOL_SOCKET, socket.SO_REUSEADDR, 1)
        try:
            s.bind((host, port))
            return True
        except OSError:
            return False


def find_free_ports(count: int = 1, port_range: tuple[int, int] = (10000, 60000), exclude: set | None = None) -> list[int]:
    exclude = set(exclude or ())
    out: list[int] = []
    tries = 0
    while len(out) < count:
        tries += 1
        if tries > 10000:
            raise RuntimeError("no free port found")
        p = random.randint(*port_range)
        if p in exclude or p in out:
            continue
        if is_port_free(p):
            out.append(p)
    return out


def find_free_port(**kw) -> int:
    return find_free_ports(1, **kw)[0]
