"""Driver side of the launcher's RPC pair: tasks (one per host) register
their addresses here, fetch each other's, and report which of the next
task's interfaces they could reach. Parity:
horovod/runner/common/service/driver_service.py:22-260."""
import threading

from horovod_b200.runner.common import network


class RegisterTaskRequest:
    def __init__(self, index, task_addresses, host_hash):
        self.index = index
        self.task_addresses = task_addresses
        self.host_hash = host_hash


class AllTaskAddressesRequest:
    def __init__(self, index):
        self.index = index


class AllTaskAddressesResponse:
    def __init__(self, all_task_addresses):
        self.all_task_addresses = all_task_addresses


class RegisterTaskToTaskAddressesRequest:
    def __init__(self, index, task_addresses):
        self.index = index
        self.task_addresses = task_addresses


class BasicDriverService(network.BasicService):
    def __init__(self, num_proc, name, key, nics=None):
        super().__init__(name, key, nics)
        self._num_proc = num_proc
        self._all_task_addresses = {}
        self._task_addresses_for_driver = {}
        self._task_addresses_for_tasks = {}
        self._task_index_host_hash = {}
        self._task_host_hash_indices = {}
        self._wait_cond = threading.Condition()

    def _handle(self, req, client_address):
        if isinstance(req, RegisterTaskRequest):
            with self._wait_cond:
                assert 0 <= req.index < self._num_proc
                self._all_task_addresses[req.index] = req.task_addresses
                # Which of the task's addresses the driver can route to: the ones on
                # the interface the registration arrived from.
                self._task_addresses_for_driver[req.index] = \
                    self._filter_by_ip(req.task_addresses, client_address[0])
                self._task_index_host_hash[req.index] = req.host_hash
                self._task_host_hash_indices.setdefault(req.host_hash, []).append(req.index)
                self._task_host_hash_indices[req.host_hash].sort()
                self._wait_cond.notify_all()
            return network.AckResponse()
        if isinstance(req, AllTaskAddressesRequest):
            return AllTaskAddressesResponse(self._all_task_addresses[req.index])
        if isinstance(req, RegisterTaskToTaskAddressesRequest):
            with self._wait_cond:
                self._task_addresses_for_tasks[req.index] = req.task_addresses
                self._wait_cond.notify_all()
            return network.AckResponse()
        return super()._handle(req, client_address)

    @staticmethod
    def _filter_by_ip(addresses, ip):
        for intf, intf_addresses in addresses.items():
            for address in intf_addresses:
                if address[0] == ip:
                    return {intf: [tuple(a) for a in intf_addresses]}
        return {k: [tuple(a) for a in v] for k, v in addresses.items()}

    def all_task_addresses(self, index):
        with self._wait_cond:
            return dict(self._all_task_addresses[index])

    def task_addresses_for_driver(self, index):
        with self._wait_cond:
            return dict(self._task_addresses_for_driver[index])

    def task_addresses_for_tasks(self, index):
        with self._wait_cond:
            return dict(self._task_addresses_for_tasks[index])

    def task_host_hash_indices(self):
        with self._wait_cond:
            return {k: list(v) for k, v in self._task_host_hash_indices.items()}

    def wait_for_initial_registration(self, timeout):
        with self._wait_cond:
            while len(self._all_task_addresses) < self._num_proc:
                self._wait_cond.wait(timeout.remaining())
                timeout.check_time_out_for("tasks to start")

    def wait_for_task_to_task_address_updates(self, timeout):
        with self._wait_cond:
            while len(self._task_addresses_for_tasks) < self._num_proc:
                self._wait_cond.wait(timeout.remaining())
                timeout.check_time_out_for("tasks to update task-to-task addresses")


class BasicDriverClient(network.BasicClient):
    def __init__(self, name, driver_addresses, key, verbose=0, match_intf=False):
        super().__init__(name, driver_addresses, key, verbose, match_intf=match_intf)

    def register_task(self, index, task_addresses, host_hash):
        self._send(RegisterTaskRequest(index, task_addresses, host_hash))

    def all_task_addresses(self, index):
        return self._send(AllTaskAddressesRequest(index)).all_task_addresses

    def register_task_to_task_addresses(self, index, task_addresses):
        self._send(RegisterTaskToTaskAddressesRequest(index, task_addresses))
