"""Addresses of this host and which of a job's hosts are this one.
Parity: horovod/runner/util/network.py (find_port lives in
horovod_b200/runner/common/network.py and is re-exported here)."""
import functools
import socket

from horovod_b200.runner.common.network import find_port  # noqa: F401
from horovod_b200.runner.util import threads


def _interfaces():
    """{interface: [IPv4 address, ...]}; empty when psutil cannot tell."""
    try:
        import psutil
    except ImportError:
        return {}
    found = {}
    for name, infos in psutil.net_if_addrs().items():
        ips = [i.address for i in infos if i.family == socket.AF_INET]
        if ips:
            found[name] = ips
    return found


@functools.lru_cache(maxsize=None)
def get_local_host_addresses():
    """Every IPv4 address configured on this machine."""
    addresses = {ip for ips in _interfaces().values() for ip in ips}
    return addresses or {"127.0.0.1"}


def get_local_intfs(nic=None):
    """Interfaces that carry the loopback address (optionally only ``nic``)."""
    return {name for name, ips in _interfaces().items()
            if "127.0.0.1" in ips and (nic is None or name == nic)}


def resolve_host_address(host_name):
    try:
        return socket.gethostbyname(host_name)
    except socket.gaierror:
        return None


def filter_local_addresses(all_host_names):
    """The host names that are NOT this machine (names that do not resolve
    count as remote), in their original order."""
    local = get_local_host_addresses()
    resolved = threads.execute_function_multithreaded(resolve_host_address,
                                                      [[h] for h in all_host_names])
    return [name for i, name in enumerate(all_host_names)
            if not resolved[i] or resolved[i] not in local]


def get_driver_ip(nics):
    """An IPv4 address of the first interface of ``nics`` (the interfaces all
    workers can reach the driver on)."""
    iface = list(nics)[0]
    ips = _interfaces().get(iface, [])
    if not ips:
        raise RuntimeError("Cannot find an IPv4 address of the common interface.")
    return ips[-1]
