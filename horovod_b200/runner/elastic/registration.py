"""Tracks what every worker of the current rendezvous round reported (ready,
success, failure) and decides, once all have reported, whether the job ends,
or a new round starts without the hosts that failed.

Parity: horovod/runner/elastic/registration.py:28-173.
"""
import logging
import threading
from collections import defaultdict

READY, SUCCESS, FAILURE = "READY", "SUCCESS", "FAILURE"


class WorkerStateRegistry:
    def __init__(self, driver, host_manager, reset_limit=None, verbose=False):
        self._driver = driver
        self._host_manager = host_manager
        self._reset_limit = reset_limit
        self._reset_count = 0
        self._lock = threading.Lock()
        self._states = {}
        self._workers = defaultdict(set)
        self._barrier = None
        self._rendezvous_id = 0
        self._verbose = verbose
        self._size = 0

    def get_recorded_slots(self):
        return list(self._states.keys())

    def get(self, state):
        return self._workers[state]

    def count(self, state):
        return len(self._workers[state])

    def reset(self, size):
        with self._lock:
            self._states.clear()
            self._workers.clear()
            self._barrier = threading.Barrier(parties=size, action=self._action)
            self._rendezvous_id += 1
            self._size = size

    def size(self):
        return self._size

    def last_rendezvous(self):
        return self._rendezvous_id

    def record_ready(self, host, slot):
        return self._record_state(host, slot, READY)

    def record_success(self, host, slot):
        return self._record_state(host, slot, SUCCESS)

    def record_failure(self, host, slot):
        return self._record_state(host, slot, FAILURE)

    def _record_state(self, host, slot, state):
        if self._driver.finished():
            return self._rendezvous_id
        if self._host_manager.is_blacklisted(host):
            return self._rendezvous_id
        key = (host, slot)
        with self._lock:
            if key in self._states:
                if state == FAILURE:
                    # A worker that already reported may still fail later;
                    # keep the failure (it blacklists the host).
                    self._workers[self._states[key]].discard(key)
                    self._states[key] = state
                    self._workers[state].add(key)
                    return self._rendezvous_id
                if self._states[key] == state:
                    return self._rendezvous_id
                # e.g. READY after SUCCESS of an earlier wave: wait like anyone.
                self._barrier.reset()
            self._states[key] = state
            self._workers[state].add(key)
            rendezvous_id = self._rendezvous_id
            barrier = self._barrier
        return self._wait(key, state, rendezvous_id, barrier)

    def _wait(self, key, state, rendezvous_id, barrier):
        while True:
            try:
                barrier.wait()
                return rendezvous_id
            except threading.BrokenBarrierError:
                if barrier.broken:
                    # Somebody recorded a change; everyone retries unless a
                    # new round has begun.
                    with self._lock:
                        if rendezvous_id != self._rendezvous_id:
                            return self._rendezvous_id
                        barrier = self._barrier
                    if barrier.broken:
                        with self._lock:
                            if self._barrier.broken:
                                self._barrier.reset()
                            barrier = self._barrier

    def _action(self):
        """Runs on one thread when every worker of the round has reported."""
        self._on_workers_recorded()

    def _on_workers_recorded(self):
        logging.info("all %d workers recorded", self.size())
        # All succeeded, or any succeeded: training is over.
        if self.count(SUCCESS) > 0:
            logging.info("at least one worker finished successfully: stopping the job")
            self._driver.stop()
            return
        if self.count(FAILURE) == self._size and self._size > 0:
            self._driver.stop(error_message="all workers failed")
            return
        # Failed hosts are not used again.
        failed_hosts = set()
        for host, slot in self.get(FAILURE):
            self._host_manager.blacklist(host)
            failed_hosts.add(host)
        if failed_hosts and all(self._host_manager.is_blacklisted(h)
                                for h in self._host_manager.current_hosts.host_slots):
            self._driver.stop(error_message="all hosts are blacklisted")
            return
        if self._reset_limit is not None and self._reset_count >= self._reset_limit:
            self._driver.stop(error_message="Job has been reset %d times, which exceeds "
                                            "the reset limit of %d" % (self._reset_count,
                                                                       self._reset_limit))
            return
        try:
            self._reset_count += 1
            self._driver.resume()
        except Exception as e:  # noqa: BLE001
            logging.exception("failed to start the next rendezvous round")
            self._driver.stop(error_message=str(e))
