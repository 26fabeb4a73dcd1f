"""Task side of the launcher's RPC pair: one service per host that the
driver (and the neighbouring task) can ping, told by the driver when every
task has registered. Parity:
horovod/runner/common/service/task_service.py:26-330 (the command-running
requests of the Spark path are not needed here: ranks are started over ssh)."""
import threading

from horovod_b200.runner.common import network


class NotifyInitialRegistrationCompleteRequest:
    pass


class ReleaseRequest:
    """The driver has everything it needs: the task service may stop."""


class BasicTaskService(network.BasicService):
    def __init__(self, name, index, key, nics=None):
        super().__init__(name, key, nics)
        self._index = index
        self._initial_registration_complete = False
        self._released = False
        self._wait_cond = threading.Condition()

    def _handle(self, req, client_address):
        if isinstance(req, NotifyInitialRegistrationCompleteRequest):
            with self._wait_cond:
                self._initial_registration_complete = True
                self._wait_cond.notify_all()
            return network.AckResponse()
        if isinstance(req, ReleaseRequest):
            with self._wait_cond:
                self._released = True
                self._wait_cond.notify_all()
            return network.AckResponse()
        return super()._handle(req, client_address)

    def wait_for_release(self, timeout):
        """Returns once the driver released this task (or the time ran out)."""
        with self._wait_cond:
            while not self._released and timeout.remaining() > 0:
                self._wait_cond.wait(min(1.0, timeout.remaining()))

    def wait_for_initial_registration(self, timeout):
        with self._wait_cond:
            while not self._initial_registration_complete:
                self._wait_cond.wait(timeout.remaining())
                timeout.check_time_out_for("tasks to start")


class BasicTaskClient(network.BasicClient):
    def __init__(self, service_name, task_addresses, key, verbose=0, match_intf=False,
                 attempts=3):
        super().__init__(service_name, task_addresses, key, verbose, match_intf=match_intf,
                         attempts=attempts)

    def notify_initial_registration_complete(self):
        self._send(NotifyInitialRegistrationCompleteRequest())

    def release(self):
        self._send(ReleaseRequest())
