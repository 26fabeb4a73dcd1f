"""Driver side of the launcher's RPC pair used for NIC discovery.

One task service runs per host. Each task tells the driver where it listens
(``register_task``), asks where its ring neighbour listens
(``all_task_addresses``), probes the neighbour on every interface and reports
the subset that answered (``register_task_to_task_addresses``). The driver
keeps one record per task and lets the launcher wait until all tasks have
registered, and later until all probe reports are in.

The RPC surface follows horovod/runner/common/service/driver_service.py:22-260
(same three calls, same waits); here one tagged message carries all three
calls and one record per task holds everything known about it.
"""
import threading

from horovod_b200.runner.common import network

# Message kinds.
REGISTER, LOOKUP, PROBE_REPORT = "register", "lookup", "probe_report"


class TaskMessage:
    """``kind`` selects the call; ``index`` is the task it concerns."""

    def __init__(self, kind, index, addresses=None, host_hash=None):
        self.kind = kind
        self.index = index
        self.addresses = addresses
        self.host_hash = host_hash


class AddressesReply:
    def __init__(self, addresses):
        self.addresses = addresses


class _TaskRecord:
    def __init__(self):
        self.listening = None     # every address the task listens on, by interface
        self.from_driver = None   # the part of them the driver can route to
        self.from_peer = None     # the part its ring predecessor could reach
        self.host_hash = None


def _as_tuples(addresses):
    return {nic: [tuple(a) for a in addrs] for nic, addrs in addresses.items()}


def _interface_of(addresses, ip):
    """The interface entry that contains ``ip`` (the registration arrived
    through it, so the driver can reach the task there); everything when the
    source address is not one the task listed (NAT, loopback aliases)."""
    for nic, addrs in addresses.items():
        if any(a[0] == ip for a in addrs):
            return {nic: [tuple(a) for a in addrs]}
    return _as_tuples(addresses)


class BasicDriverService(network.BasicService):
    def __init__(self, num_proc, name, key, nics=None):
        super().__init__(name, key, nics)
        self._num_proc = num_proc
        self._tasks = {}
        self._changed = threading.Condition()

    def _record(self, index):
        if not 0 <= index < self._num_proc:
            raise ValueError("task index %r out of range (0..%d)" % (index, self._num_proc - 1))
        return self._tasks.setdefault(index, _TaskRecord())

    def _handle(self, req, client_address):
        if not isinstance(req, TaskMessage):
            return super()._handle(req, client_address)
        with self._changed:
            if req.kind == LOOKUP:
                return AddressesReply(self._tasks[req.index].listening)
            rec = self._record(req.index)
            if req.kind == REGISTER:
                rec.listening = req.addresses
                rec.from_driver = _interface_of(req.addresses, client_address[0])
                rec.host_hash = req.host_hash
            elif req.kind == PROBE_REPORT:
                rec.from_peer = req.addresses
            else:
                raise ValueError("unknown task message %r" % req.kind)
            self._changed.notify_all()
        return network.AckResponse()

    # ---- what the launcher reads ----------------------------------------------
    def all_task_addresses(self, index):
        with self._changed:
            return dict(self._tasks[index].listening)

    def task_addresses_for_driver(self, index):
        with self._changed:
            return dict(self._tasks[index].from_driver)

    def task_addresses_for_tasks(self, index):
        with self._changed:
            return dict(self._tasks[index].from_peer)

    def task_host_hash_indices(self):
        """host hash -> sorted indices of the tasks that run on that host."""
        with self._changed:
            by_host = {}
            for index in sorted(self._tasks):
                rec = self._tasks[index]
                if rec.listening is not None:
                    by_host.setdefault(rec.host_hash, []).append(index)
            return by_host

    def _wait_until_all(self, have, timeout, activity):
        with self._changed:
            while sum(1 for r in self._tasks.values() if have(r)) < self._num_proc:
                self._changed.wait(timeout.remaining())
                timeout.check_time_out_for(activity)

    def wait_for_initial_registration(self, timeout):
        self._wait_until_all(lambda r: r.listening is not None, timeout, "tasks to start")

    def wait_for_task_to_task_address_updates(self, timeout):
        self._wait_until_all(lambda r: r.from_peer is not None, timeout,
                             "tasks to update task-to-task addresses")


class BasicDriverClient(network.BasicClient):
    def __init__(self, name, driver_addresses, key, verbose=0, match_intf=False):
        super().__init__(name, driver_addresses, key, verbose, match_intf=match_intf)

    def register_task(self, index, task_addresses, host_hash):
        self._send(TaskMessage(REGISTER, index, task_addresses, host_hash))

    def all_task_addresses(self, index):
        return self._send(TaskMessage(LOOKUP, index)).addresses

    def register_task_to_task_addresses(self, index, task_addresses):
        self._send(TaskMessage(PROBE_REPORT, index, task_addresses))
