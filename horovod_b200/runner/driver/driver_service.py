"""NIC discovery for multi-host jobs: which network interfaces are routed
between all hosts. One task service is started per host; each registers with
the driver, then probes every interface of the next host's task (a ring) and
reports the ones that answered; the interfaces common to all reports are the
ones handed to the ranks (HOROVOD_GLOO_IFACE / NCCL_SOCKET_IFNAME).
Parity: horovod/runner/driver/driver_service.py:30-260,
horovod/runner/task_fn.py:23-67."""
import os
import sys
import threading

from horovod_b200.runner.common import safe_shell_exec, secret
from horovod_b200.runner.common.hosts import host_hash as _host_hash
from horovod_b200.runner.common.service import driver_service, task_service
from horovod_b200.runner.common.timeout import Timeout


class HorovodRunDriverService(driver_service.BasicDriverService):
    NAME = "horovod driver service"

    def __init__(self, num_hosts, key, nics=None):
        super().__init__(num_hosts, HorovodRunDriverService.NAME, key, nics)


class HorovodRunDriverClient(driver_service.BasicDriverClient):
    def __init__(self, driver_addresses, key, verbose=0, match_intf=False):
        super().__init__(HorovodRunDriverService.NAME, driver_addresses, key, verbose,
                         match_intf=match_intf)


class HorovodRunTaskService(task_service.BasicTaskService):
    NAME_FORMAT = "horovod task service #%d"

    def __init__(self, index, key, nics=None):
        super().__init__(HorovodRunTaskService.NAME_FORMAT % index, index, key, nics)


class HorovodRunTaskClient(task_service.BasicTaskClient):
    def __init__(self, index, task_addresses, key, verbose=0, match_intf=False, attempts=3):
        super().__init__(HorovodRunTaskService.NAME_FORMAT % index, task_addresses, key,
                         verbose, match_intf=match_intf, attempts=attempts)


def task_fn(index, num_hosts, driver_addresses, key, nics=None, start_timeout_s=30,
            host_hash=None):
    """What runs on each host: register, wait for the others, probe the next
    host's interfaces, report, and stay up until the previous host has probed
    this one (the driver's wait covers that)."""
    timeout = Timeout(start_timeout_s, "Timed out waiting for {activity}.")
    task = HorovodRunTaskService(index, key, nics)
    try:
        driver = HorovodRunDriverClient(driver_addresses, key)
        driver.register_task(index, task.addresses(), host_hash or _host_hash())
        task.wait_for_initial_registration(timeout)
        next_index = (index + 1) % num_hosts
        next_addresses = driver.all_task_addresses(next_index)
        # Only the interfaces on which the neighbour actually answers count.
        next_client = HorovodRunTaskClient(next_index, next_addresses, key, match_intf=True,
                                           attempts=2)
        driver.register_task_to_task_addresses(next_index, next_client.addresses())
        # The previous host may still be probing this one: stay up until the
        # driver has heard from everybody.
        task.wait_for_release(timeout)
    finally:
        task.shutdown()


def _launch_task_servers(all_host_names, local_host_names, driver_addresses, key, nics,
                         ssh_port=None, ssh_identity_file=None, verbose=0):
    """Starts task_fn on every host (a thread for this host, ssh elsewhere)."""
    import base64
    import cloudpickle
    threads = []
    num_hosts = len(all_host_names)
    for index, host in enumerate(all_host_names):
        if host in local_host_names:
            t = threading.Thread(target=task_fn, daemon=True,
                                 args=(index, num_hosts, driver_addresses, key, nics))
        else:
            payload = base64.b64encode(cloudpickle.dumps(
                (index, num_hosts, driver_addresses, key, nics))).decode()
            ssh = "ssh -o PasswordAuthentication=no -o StrictHostKeyChecking=no"
            if ssh_port:
                ssh += " -p %d" % ssh_port
            if ssh_identity_file:
                ssh += " -i %s" % ssh_identity_file
            command = "%s %s '%s -m horovod_b200.runner.driver.driver_service %s'" % (
                ssh, host, sys.executable, payload)
            t = threading.Thread(target=safe_shell_exec.execute, daemon=True,
                                 args=(command,), kwargs={"env": dict(os.environ)})
        t.start()
        threads.append(t)
    return threads


def get_common_interfaces(all_host_names, local_host_names=("localhost", "127.0.0.1"),
                          nics=None, start_timeout_s=30, ssh_port=None, ssh_identity_file=None,
                          verbose=0):
    """Names of the interfaces over which every host reaches the next one.
    A single-host job needs no probing: loopback (or ``nics``) is returned."""
    remote = [h for h in all_host_names if h not in local_host_names]
    if not remote:
        return set(nics) if nics else {"lo"}
    key = secret.make_secret_key()
    num_hosts = len(all_host_names)
    driver = HorovodRunDriverService(num_hosts, key, nics)
    try:
        _launch_task_servers(all_host_names, local_host_names, driver.addresses(), key, nics,
                             ssh_port, ssh_identity_file, verbose)
        return _run_probe(driver, key, num_hosts, start_timeout_s)
    finally:
        driver.shutdown()


def _run_probe(driver, key, num_hosts, start_timeout_s=30):
    """Driver half of the probe; the tasks must already be starting."""
    timeout = Timeout(start_timeout_s, "Timed out waiting for {activity}. Check that every "
                                       "host can reach the launcher and the next host.")
    driver.wait_for_initial_registration(timeout)
    clients = []
    for index in range(num_hosts):
        client = HorovodRunTaskClient(index, driver.task_addresses_for_driver(index), key)
        client.notify_initial_registration_complete()
        clients.append(client)
    driver.wait_for_task_to_task_address_updates(timeout)
    for client in clients:
        try:
            client.release()
        except Exception:  # noqa: BLE001 - a task that already left is fine
            pass
    common = None
    for index in range(num_hosts):
        reachable = set(driver.task_addresses_for_tasks(index).keys())
        common = reachable if common is None else common & reachable
    if not common:
        raise Exception("Unable to find a set of common task-to-task communication interfaces: %s"
                        % [(i, driver.task_addresses_for_tasks(i)) for i in range(num_hosts)])
    return common


if __name__ == "__main__":
    # Remote entry point: python -m horovod_b200.runner.driver.driver_service <payload>
    import base64
    import cloudpickle
    task_fn(*cloudpickle.loads(base64.b64decode(sys.argv[1])))
