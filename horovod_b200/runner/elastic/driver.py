"""Elastic driver: keeps the running workers in line with what host discovery
reports. A discovery thread polls once a second; when hosts appear or
disappear the driver tells the current rank 0 (through its notification
service), the workers raise HostsUpdatedInterrupt at their next commit and
come back to the rendezvous server, and a new round of slot assignments is
published. Failed workers blacklist their host and also trigger a new round.

Parity: horovod/runner/elastic/driver.py:30-313.
"""
import logging
import queue
import threading
import time
from collections import defaultdict

from horovod_b200.common.elastic import HostUpdateResult
from horovod_b200.runner.common import hosts
from horovod_b200.runner.elastic.discovery import HostManager
from horovod_b200.runner.elastic.registration import WorkerStateRegistry
from horovod_b200.runner.elastic.worker import WorkerNotificationClient

DISCOVER_HOSTS_FREQUENCY_SECS = 1.0
ELASTIC_TIMEOUT_SECS = 600


def _epoch_time_s():
    return int(time.time())


class Results:
    def __init__(self, error_message, worker_results):
        self.error_message = error_message
        self.worker_results = worker_results


class ResultsRecorder:
    def __init__(self):
        self._error_message = None
        self._worker_results = {}
        self._worker_threads = queue.Queue()

    def expect(self, worker_thread):
        self._worker_threads.put(worker_thread)

    def set_error_message(self, error_message):
        self._error_message = error_message

    def add_result(self, key, value):
        if key in self._worker_results:
            return
        self._worker_results[key] = value

    def get_results(self):
        while not self._worker_threads.empty():
            self._worker_threads.get().join()
        return Results(self._error_message, self._worker_results)


class ElasticDriver:
    def __init__(self, rendezvous, discovery, min_np, max_np, timeout=None, reset_limit=None,
                 verbose=0):
        self._rendezvous = rendezvous
        self._host_manager = HostManager(discovery)
        self._min_np = min_np
        self._max_np = max_np
        self._verbose = verbose

        self._host_assignments = {}
        self._rank_assignments = {}
        self._world_size = 0
        self._round = 0

        self._wait_hosts_cond = threading.Condition()
        self._timeout = timeout or ELASTIC_TIMEOUT_SECS

        self._create_worker_fn = None
        self._worker_clients = {}

        self._worker_registry = WorkerStateRegistry(self, self._host_manager,
                                                    reset_limit=reset_limit)
        self._results = ResultsRecorder()
        self._shutdown = threading.Event()

        self._discovery_thread = threading.Thread(target=self._discover_hosts, daemon=True,
                                                  name="hvd-elastic-discovery")
        self._discovery_thread.start()

    @property
    def host_manager(self):
        return self._host_manager

    def start(self, np, create_worker_fn):
        self._create_worker_fn = create_worker_fn
        self._activate_workers(np)

    def resume(self):
        self._activate_workers(self._min_np)

    def stop(self, error_message=None):
        self._results.set_error_message(error_message)
        self._shutdown.set()
        self._discovery_thread.join(timeout=5)

    def finished(self):
        return self._shutdown.is_set()

    def get_results(self):
        return self._results.get_results()

    def rendezvous_round(self):
        return self._round

    def register_worker_server(self, host, slot, addresses, secret_key):
        self._worker_clients[(host, slot)] = WorkerNotificationClient(
            addresses, secret_key, self._verbose)

    def get_worker_client(self, slot_info):
        return self._worker_clients.get((slot_info.hostname, slot_info.local_rank))

    def record_ready(self, host, slot):
        self._worker_registry.record_ready(host, slot)

    def world_size(self):
        return self._world_size

    def local_size(self, host):
        return len(self._host_assignments[host])

    def get_slot_info(self, host, slot):
        if self.has_rank_assignment(host, slot):
            return self._host_assignments[host][slot]
        return hosts.INVALID_SLOT_INFO

    def get_coordinator_info(self):
        return self._rank_assignments.get(0)

    def has_rank_assignment(self, host, slot):
        if self._host_manager.is_blacklisted(host):
            return False
        return host in self._host_assignments and len(self._host_assignments[host]) > slot

    @property
    def host_assignments(self):
        return self._host_assignments

    def wait_for_available_slots(self, min_np, min_hosts=1):
        """Blocks until discovery offers at least min_np slots on at least
        min_hosts hosts; raises after the elastic timeout."""
        tmout = time.time() + self._timeout
        self._wait_hosts_cond.acquire()
        try:
            while True:
                current_hosts = self._host_manager.current_hosts
                avail_slots = current_hosts.count_available_slots()
                if avail_slots >= min_np and len(current_hosts.available_hosts) >= min_hosts:
                    return current_hosts
                if self._shutdown.is_set():
                    raise RuntimeError("Job has been shutdown, see above error messages "
                                       "for details.")
                self._wait_hosts_cond.wait(max(0.0, tmout - time.time()))
                if time.time() >= tmout:
                    raise TimeoutError(
                        "Timed out waiting for the minimum number of slots (%d) to become "
                        "available; only %d are. Check that the discovery script prints "
                        "the expected hosts, or increase --elastic-timeout."
                        % (min_np, self._host_manager.current_hosts.count_available_slots()))
        finally:
            self._wait_hosts_cond.release()

    def _activate_workers(self, min_np):
        current_hosts = self.wait_for_available_slots(min_np)
        pending_slots = self._update_host_assignments(current_hosts)
        self._worker_registry.reset(self.world_size())
        self._start_worker_processes(pending_slots)

    def _discover_hosts(self):
        first_update = True
        while not self._shutdown.is_set():
            self._wait_hosts_cond.acquire()
            try:
                update_res = self._host_manager.update_available_hosts()
                if update_res != HostUpdateResult.no_update:
                    self._notify_workers_host_changes(self._host_manager.current_hosts,
                                                      update_res)
                    self._wait_hosts_cond.notify_all()
            except RuntimeError as e:
                if first_update:
                    # Misconfiguration: fail fast rather than wait out the timeout.
                    self._shutdown.set()
                    self._wait_hosts_cond.notify_all()
                    raise
                logging.warning("host discovery failed: %s", e)
            finally:
                self._wait_hosts_cond.release()
            first_update = False
            self._shutdown.wait(DISCOVER_HOSTS_FREQUENCY_SECS)

    def _notify_workers_host_changes(self, current_hosts, update_res):
        next_host_assignments = {}
        if current_hosts.count_available_slots() >= self._min_np:
            next_host_assignments, _ = self._get_host_assignments(current_hosts)
        if next_host_assignments == self.host_assignments:
            # Same placement (e.g. only spare hosts changed): nothing to do.
            return
        coordinator_info = self.get_coordinator_info()
        if not coordinator_info:
            return
        coordinator_client = self.get_worker_client(coordinator_info)
        if not coordinator_client:
            return
        timestamp = _epoch_time_s()
        try:
            coordinator_client.notify_hosts_updated(timestamp, update_res)
        except Exception:  # noqa: BLE001
            if self._verbose >= 2:
                logging.exception("failed to notify the coordinator of a host change")

    def _get_host_assignments(self, current_hosts):
        # Hosts already in use come first so that a surviving worker gets rank 0.
        host_list = [hosts.HostInfo(host, current_hosts.get_slots(host))
                     for host in current_hosts.host_assignment_order]
        host_assignments_list = hosts.get_host_assignments(host_list, self._min_np, self._max_np)
        host_assignments = defaultdict(list)
        for slot_info in host_assignments_list:
            host_assignments[slot_info.hostname].append(slot_info)
        return dict(host_assignments), host_assignments_list

    def _update_host_assignments(self, current_hosts):
        # At least one host of the previous round must survive: the state to
        # continue from lives in its workers.
        active_hosts = set(self._host_assignments.keys())
        if active_hosts and not (active_hosts & current_hosts.available_hosts):
            raise RuntimeError("No hosts from previous set remaining, unable to broadcast "
                               "state.")
        self._host_assignments, host_assignments_list = self._get_host_assignments(current_hosts)
        if self._host_assignments:
            self._world_size = len(host_assignments_list)
            self._round += 1
            self._rendezvous.init(host_assignments_list)
        self._rank_assignments = {s.rank: s for s in host_assignments_list}
        # Slots that have no running worker yet.
        pending = []
        for slot_info in host_assignments_list:
            key = (slot_info.hostname, slot_info.local_rank)
            if key not in getattr(self, "_running", set()):
                pending.append(slot_info)
        return pending

    def _start_worker_processes(self, pending_slots):
        if not hasattr(self, "_running"):
            self._running = set()
        for slot_info in pending_slots:
            self._start_worker_process(slot_info)

    def _start_worker_process(self, slot_info):
        create_worker_fn = self._create_worker_fn
        shutdown_event = self._shutdown
        host_event = self._host_manager.get_host_event(slot_info.hostname)
        key = (slot_info.hostname, slot_info.local_rank)
        self._running.add(key)

        def run_worker():
            res = create_worker_fn(slot_info, [shutdown_event, host_event])
            exit_code, timestamp = res if isinstance(res, tuple) else (res, _epoch_time_s())
            self._running.discard(key)
            self._handle_worker_exit(slot_info, exit_code, timestamp)

        thread = threading.Thread(target=run_worker, daemon=True,
                                  name="hvd-worker-%s-%d" % key)
        thread.start()
        self._results.expect(thread)

    def _handle_worker_exit(self, slot_info, exit_code, timestamp):
        if not self.has_rank_assignment(slot_info.hostname, slot_info.local_rank):
            # Worker of a host that was removed or blacklisted: not a result.
            return
        if exit_code == 0:
            rendezvous_id = self._worker_registry.record_success(slot_info.hostname,
                                                                 slot_info.local_rank)
        else:
            rendezvous_id = self._worker_registry.record_failure(slot_info.hostname,
                                                                 slot_info.local_rank)
        if self.finished() and self._worker_registry.last_rendezvous() == rendezvous_id:
            name = "%s[%d]" % (slot_info.hostname, slot_info.local_rank)
            self._results.add_result(name, (exit_code, timestamp))
