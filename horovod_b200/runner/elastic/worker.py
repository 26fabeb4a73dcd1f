"""Worker side of host-change notification: each elastic worker runs a small
service; the driver calls it when the set of hosts changes, and the message
ends up in every registered State's queue (checked at the next commit).

Parity: horovod/runner/elastic/worker.py:32-119.
"""
import os
import pickle
import socket
import urllib.request

from horovod_b200.runner.common import network, secret

PUT_WORKER_ADDRESSES = "worker_addresses"


class HostsUpdatedRequest:
    """Sent by the driver when discovery reported a change."""

    def __init__(self, timestamp, res):
        self.timestamp = timestamp
        self.res = res


class WorkerNotificationService(network.BasicService):
    NAME = "worker notification service"

    def __init__(self, key, nic, manager):
        super().__init__(WorkerNotificationService.NAME, key, nic)
        self._manager = manager

    def _handle(self, req, client_address):
        if isinstance(req, HostsUpdatedRequest):
            self._manager.handle_hosts_updated(req.timestamp, req.res)
            return network.AckResponse()
        return super()._handle(req, client_address)


class WorkerNotificationClient(network.BasicClient):
    def __init__(self, addresses, key, verbose=0, match_intf=False):
        super().__init__(WorkerNotificationService.NAME, addresses, key, verbose,
                         match_intf=match_intf, probe_timeout=5, attempts=2)

    def notify_hosts_updated(self, timestamp, update_res):
        self._send(HostsUpdatedRequest(timestamp, update_res))


def start_notification_service(manager):
    """Starts the service and registers its address with the driver's
    rendezvous server. Returns the service, or None outside elastic jobs."""
    addr = os.environ.get("HOROVOD_GLOO_RENDEZVOUS_ADDR")
    port = os.environ.get("HOROVOD_GLOO_RENDEZVOUS_PORT")
    if os.environ.get("HOROVOD_ELASTIC") != "1" or not addr or not port:
        return None
    key = secret.make_secret_key()
    service = WorkerNotificationService(key, os.environ.get("HOROVOD_GLOO_IFACE"), manager)
    host = os.environ.get("HOROVOD_HOSTNAME", socket.gethostname())
    local_rank = os.environ.get("HOROVOD_LOCAL_RANK", "0")
    payload = pickle.dumps((service.addresses(), key))
    req = urllib.request.Request(
        "http://%s:%s/%s/%s:%s" % (addr, port, PUT_WORKER_ADDRESSES, host, local_rank),
        data=payload, method="PUT")
    with urllib.request.urlopen(req, timeout=30):
        pass
    return service
