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


# --------------------------------------------------------------------------- host:port strings, IPv6 aware
def is_ipv6_literal(host: str) -> bool:
    """True for an IPv6 address literal (brackets and a ``%zone`` suffix allowed)."""
    import ipaddress

    h = host[1:-1] if host.startswith("[") and host.endswith("]") else host
    try:
        return ipaddress.ip_address(h.split("%", 1)[0]).version == 6
    except ValueError:
        return False


def format_hostport(host: str, port: int) -> str:
    """``host:port`` as it goes into a URL: IPv6 literals get brackets (``[fe80::1]:8000``)."""
    h = host if not is_ipv6_literal(host) or host.startswith("[") else f"[{host}]"
    return f"{h}:{int(port)}"


def split_hostport(addr: str) -> tuple[str, int]:
    """Inverse of :func:`format_hostport`. Accepts ``name:port``, ``1.2.3.4:port``, ``[v6]:port`` and, because it is
    unambiguous when the last group is a valid port and the rest a valid address, the unbracketed ``v6:port`` that some
    launchers write. Reference: ``areal/utils/network.py`` (``split_hostport``), ``tests/test_network_ipv6_utils.py``."""
    import ipaddress

    addr = addr.strip()
    if addr.startswith("["):
        end = addr.find("]")
        if end < 0 or not addr[end + 1:].startswith(":"):
            raise ValueError(f"invalid bracketed address '{addr}'")
        host, port = addr[1:end], addr[end + 2:]
        if not is_ipv6_literal(host):
            raise ValueError(f"invalid bracketed address '{addr}'")
    else:
        host, sep, port = addr.rpartition(":")
        if not sep or not host:
            raise ValueError(f"address '{addr}' has no port")
        if ":" in host:                                  # unbracketed IPv6 followed by a port
            try:
                ipaddress.ip_address(host.split("%", 1)[0])
            except ValueError as e:
                raise ValueError(f"invalid address '{addr}'") from e
    if not port.isdigit() or not 0 <= int(port) <= 65535:
        raise ValueError(f"invalid port in '{addr}'")
    return host, int(port)


def gethostip_any() -> str:
    """This host's outward address: the IPv4 route if there is one, else the IPv6 route, else loopback."""
    for fam, probe in ((socket.AF_INET, ("10.255.255.255", 1)), (socket.AF_INET6, ("2001:db8::1", 1))):
        try:
            with closing(socket.socket(fam, socket.SOCK_DGRAM)) as s:
                s.connect(probe)
                ip = s.getsockname()[0]
                if ip and ip not in ("0.0.0.0", "::"):
                    return ip
        except OSError:
            continue
    return "127.0.0.1"
