"""Host-list parsing and local interface lookup for the launcher
(role of bluefog/run/network_util.py:30-219, without the ssh checks of a multi-host job)."""
import socket

import psutil

_LOCAL_NAMES = {"localhost", "127.0.0.1", "::1"}


def parse_hosts(spec: str):
    """'a:2,b:4' -> [('a', 2), ('b', 4)]; a missing slot count means 1."""
    out = []
    for item in spec.split(","):
        item = item.strip()
        if not item:
            continue
        name, _, slots = item.partition(":")
        out.append((name, int(slots) if slots else 1))
    return out


def parse_hostfile(path: str):
    """Lines of the form 'hostname slots=N' (comments with #)."""
    out = []
    with open(path) as f:
        for line in f:
            line = line.split("#", 1)[0].strip()
            if not line:
                continue
            parts = line.split()
            slots = 1
            for p in parts[1:]:
                if p.startswith("slots="):
                    slots = int(p[len("slots="):])
            out.append((parts[0], slots))
    return out


def local_addresses():
    addrs = set(_LOCAL_NAMES)
    for infos in psutil.net_if_addrs().values():
        for info in infos:
            if info.family in (socket.AF_INET, socket.AF_INET6):
                addrs.add(info.address.split("%")[0])
    addrs.add(socket.gethostname())
    return addrs


def is_local_host(name: str) -> bool:
    if name in local_addresses():
        return True
    try:
        return socket.gethostbyname(name) in local_addresses()
    except OSError:
        return False


def interface_address(nic: str) -> str:
    """IPv4 address of a named interface."""
    infos = psutil.net_if_addrs().get(nic)
    if not infos:
        raise SystemExit(f"bfrun: unknown network interface {nic!r}; available: "
                         + ", ".join(sorted(psutil.net_if_addrs())))
    for info in infos:
        if info.family == socket.AF_INET:
            return info.address
    raise SystemExit(f"bfrun: interface {nic!r} has no IPv4 address")
