"""Elastic driver: one membership state machine for the whole job.

The job lives through numbered *rounds*. A round is a fixed placement of
ranks on slots, published to the rendezvous server. Every worker of a round
eventually *reports* once: READY (it came back to the rendezvous because
something changed), SUCCESS or FAILURE (its process ended). When the last
report of a round is in, exactly one thread takes the decision for everybody:

  any SUCCESS              -> the job is over, fine
  everybody FAILED         -> the job is over, with an error
  otherwise                -> hosts of failed workers are banned and, unless
                              the reset limit is spent, the next round starts
                              on whatever hosts discovery offers now

while all other reporters sleep on one condition variable until the round
number moves on or the job ends. A background thread polls host discovery
once a second; when the placement would change it pings the notification
service of the current rank 0, whose ``State.commit()`` then makes all workers
come back (READY) and so closes the round.

Behaviour follows horovod/runner/elastic/driver.py:30-313 and
registration.py:28-173 (older hosts first so that a surviving worker becomes
rank 0; at least one host of the previous round must survive; workers are
started only on slots that have none; results are kept for the workers of the
final round). The structure differs: the reference splits this between a
driver, a registry and a threading.Barrier with an action callback.
"""
import collections
import enum
import logging
import threading
import time

from horovod_b200.common.elastic import HostUpdateResult
from horovod_b200.runner.common import hosts as host_math
from horovod_b200.runner.elastic.discovery import HostManager
from horovod_b200.runner.elastic.worker import WorkerNotificationClient

DISCOVER_HOSTS_FREQUENCY_SECS = 1.0
ELASTIC_TIMEOUT_SECS = 600

JobOutcome = collections.namedtuple("JobOutcome", ["error_message", "worker_results"])


class Report(enum.Enum):
    READY = "READY"
    SUCCESS = "SUCCESS"
    FAILURE = "FAILURE"


class _Round:
    """Placement of one round and the reports received for it."""

    def __init__(self, number, slots):
        self.number = number
        self.slots = list(slots)
        self.by_host = collections.defaultdict(list)
        for s in self.slots:
            self.by_host[s.hostname].append(s)
        self.by_rank = {s.rank: s for s in self.slots}
        self.reports = {}       # (host, local_rank) -> Report
        self.deciding = False   # the last reporter is working out what comes next

    def slot(self, host, local_rank):
        on_host = self.by_host.get(host, ())
        return on_host[local_rank] if local_rank < len(on_host) else None

    def complete(self):
        return len(self.reports) >= len(self.slots) > 0

    def placement(self):
        return {h: list(v) for h, v in self.by_host.items()}


class ElasticDriver:
    def __init__(self, rendezvous, discovery, min_np, max_np, timeout=None, reset_limit=None,
                 verbose=0):
        self._rendezvous = rendezvous
        self._hosts = HostManager(discovery)
        self._min_np, self._max_np = min_np, max_np
        self._timeout = timeout or ELASTIC_TIMEOUT_SECS
        self._reset_limit = reset_limit
        self._resets = 0
        self._verbose = verbose

        self._cv = threading.Condition()  # guards everything below
        self._round = _Round(0, [])
        self._finished = False
        self._error = None
        self._results = {}
        self._live = set()                # (host, local_rank) with a running worker
        self._threads = []
        self._spawn = None
        self._notify_clients = {}
        self._undelivered_change = HostUpdateResult.no_update
        self._stop_event = threading.Event()  # handed to workers: the job is ending

        self._poller = threading.Thread(target=self._poll_discovery, daemon=True,
                                        name="hvd-elastic-discovery")
        self._poller.start()

    # ---- what the launcher and the rendezvous handler call -------------------
    @property
    def host_manager(self):
        return self._hosts

    @property
    def host_assignments(self):
        with self._cv:
            return self._round.placement()

    def start(self, np, create_worker_fn):
        """Begins the first round with at least ``np`` slots.
        ``create_worker_fn(slot_info, events)`` runs one worker to its end and
        returns its exit code, or ``(exit code, timestamp)``."""
        self._spawn = create_worker_fn
        self._begin_round(np)

    def resume(self):
        self._begin_round(self._min_np)

    def stop(self, error_message=None):
        with self._cv:
            if not self._finished:
                self._finished = True
                self._error = error_message
            self._cv.notify_all()
        self._stop_event.set()
        if threading.current_thread() is not self._poller:
            self._poller.join(timeout=5)

    def finished(self):
        with self._cv:
            return self._finished

    def get_results(self):
        """Waits for every worker thread (also those started later on) and
        returns the outcome of the job."""
        while True:
            with self._cv:
                pending = [t for t in self._threads if t.is_alive()]
                if not pending:
                    return JobOutcome(self._error, dict(self._results))
            for t in pending:
                t.join()

    def rendezvous_round(self):
        with self._cv:
            return self._round.number

    def world_size(self):
        with self._cv:
            return len(self._round.slots)

    def local_size(self, host):
        with self._cv:
            return len(self._round.by_host[host])

    def has_rank_assignment(self, host, slot):
        if self._hosts.is_blacklisted(host):
            return False
        with self._cv:
            return self._round.slot(host, slot) is not None

    def get_slot_info(self, host, slot):
        if self._hosts.is_blacklisted(host):
            return host_math.INVALID_SLOT_INFO
        with self._cv:
            return self._round.slot(host, slot) or host_math.INVALID_SLOT_INFO

    def get_coordinator_info(self):
        with self._cv:
            return self._round.by_rank.get(0)

    def register_worker_server(self, host, slot, addresses, secret_key):
        client = WorkerNotificationClient(addresses, secret_key, self._verbose)
        with self._cv:
            self._notify_clients[(host, slot)] = client
            missed = self._undelivered_change
        if missed != HostUpdateResult.no_update:
            # Hosts changed while rank 0 could not be told yet (it had not
            # started its notification service): tell it now.
            self._placement_may_change(missed)

    def get_worker_client(self, slot_info):
        with self._cv:
            return self._notify_clients.get((slot_info.hostname, slot_info.local_rank))

    def record_ready(self, host, slot):
        """A worker is back at the rendezvous: blocks until the round it
        belonged to has been closed and returns the current round number."""
        return self._report(host, slot, Report.READY)

    def wait_for_available_slots(self, min_np, min_hosts=1):
        """Blocks until discovery offers at least ``min_np`` usable slots on at
        least ``min_hosts`` hosts and returns that view; TimeoutError after the
        elastic timeout, RuntimeError if the job ends meanwhile."""
        deadline = time.monotonic() + self._timeout
        with self._cv:
            while True:
                view = self._hosts.current_hosts
                if (view.count_available_slots() >= min_np and
                        len(view.available_hosts) >= min_hosts):
                    return view
                if self._finished:
                    raise RuntimeError("Job has been shutdown, see above error messages "
                                       "for details.")
                left = deadline - time.monotonic()
                if left <= 0:
                    raise TimeoutError(
                        "Timed out waiting for the minimum number of slots (%d) to become "
                        "available; only %d are. Check that the discovery script prints "
                        "the expected hosts, or increase --elastic-timeout."
                        % (min_np, view.count_available_slots()))
                self._cv.wait(left)

    # ---- rounds -------------------------------------------------------------
    def _plan(self, view):
        """Rank placement on the hosts of ``view``, most senior host first."""
        offered = [host_math.HostInfo(h, view.get_slots(h)) for h in view.host_assignment_order]
        return host_math.get_host_assignments(offered, self._min_np, self._max_np)

    def _begin_round(self, min_np):
        view = self.wait_for_available_slots(min_np)
        with self._cv:
            previous = set(self._round.by_host)
            if previous and not (previous & view.available_hosts):
                # The state to continue from lives in the old workers.
                raise RuntimeError("No hosts from previous set remaining, unable to "
                                   "broadcast state.")
            slots = self._plan(view)
            self._round = _Round(self._round.number + 1, slots)
            self._rendezvous.init(slots)
            unmanned = [s for s in slots if (s.hostname, s.local_rank) not in self._live]
            for s in unmanned:
                self._live.add((s.hostname, s.local_rank))
            self._cv.notify_all()
        for s in unmanned:
            self._launch(s)

    def _launch(self, slot_info):
        key = (slot_info.hostname, slot_info.local_rank)
        events = [self._stop_event, self._hosts.get_host_event(slot_info.hostname)]

        def body():
            outcome = self._spawn(slot_info, events)
            code, stamp = outcome if isinstance(outcome, tuple) else (outcome, int(time.time()))
            with self._cv:
                self._live.discard(key)
            self._worker_ended(slot_info, code, stamp)

        t = threading.Thread(target=body, daemon=True, name="hvd-worker-%s-%d" % key)
        with self._cv:
            self._threads.append(t)
        t.start()

    def _worker_ended(self, slot_info, code, stamp):
        host, slot = slot_info.hostname, slot_info.local_rank
        if not self.has_rank_assignment(host, slot):
            return  # its host was dropped or banned: not part of the outcome
        seen_round = self._report(host, slot, Report.SUCCESS if code == 0 else Report.FAILURE)
        with self._cv:
            if self._finished and seen_round == self._round.number:
                self._results.setdefault("%s[%d]" % (host, slot), (code, stamp))

    def _report(self, host, slot, what):
        key = (host, slot)
        if self._hosts.is_blacklisted(host):
            return self.rendezvous_round()
        with self._cv:
            if self._finished:
                return self._round.number
            rnd = self._round
            if rnd.slot(host, slot) is None:
                return rnd.number  # not a member of this round: nothing to wait for
            earlier = rnd.reports.get(key)
            if earlier is not None:
                if what is Report.FAILURE:
                    rnd.reports[key] = what  # a worker may fail after it reported
                    return rnd.number
                if earlier is what:
                    return rnd.number
            rnd.reports[key] = what
            if rnd.complete() and not rnd.deciding:
                rnd.deciding = True
                decide = True
            else:
                decide = False
                while self._round is rnd and not self._finished:
                    self._cv.wait()
        if decide:
            self._close(rnd)
        return rnd.number

    def _close(self, rnd):
        """Runs on the thread of the last reporter of ``rnd``."""
        statuses = list(rnd.reports.values())
        if Report.SUCCESS in statuses:
            logging.info("a worker finished successfully: the job is complete")
            self.stop()
            return
        if all(s is Report.FAILURE for s in statuses):
            self.stop(error_message="all workers failed")
            return
        for (host, _slot), status in rnd.reports.items():
            if status is Report.FAILURE:
                self._hosts.blacklist(host)
        if not self._hosts.current_hosts.available_hosts and \
                any(s is Report.FAILURE for s in statuses):
            self.stop(error_message="all hosts are blacklisted")
            return
        if self._reset_limit is not None and self._resets >= self._reset_limit:
            self.stop(error_message="Job has been reset %d times, which exceeds the reset "
                                    "limit of %d" % (self._resets, self._reset_limit))
            return
        self._resets += 1
        try:
            self.resume()
        except Exception as e:  # noqa: BLE001
            logging.exception("could not start the next rendezvous round")
            self.stop(error_message=str(e))

    # ---- discovery ------------------------------------------------------------
    def _poll_discovery(self):
        first = True
        while not self._stop_event.is_set():
            try:
                change = self._hosts.update_available_hosts()
            except RuntimeError as e:
                if first:
                    # A broken discovery script is a configuration error: end
                    # the job now instead of waiting out the timeout.
                    self.stop(error_message="host discovery failed: %s" % e)
                    raise
                logging.warning("host discovery failed: %s", e)
                change = HostUpdateResult.no_update
            first = False
            if change != HostUpdateResult.no_update:
                self._placement_may_change(change)
                with self._cv:
                    self._cv.notify_all()
            self._stop_event.wait(DISCOVER_HOSTS_FREQUENCY_SECS)

    def _placement_may_change(self, change):
        """Tells the current rank 0 about a host change, unless the ranks would
        be placed exactly as they are (e.g. only spare capacity changed)."""
        view = self._hosts.current_hosts
        planned = []
        if view.count_available_slots() >= self._min_np:
            planned = self._plan(view)
        with self._cv:
            if planned == self._round.slots:
                self._undelivered_change = HostUpdateResult.no_update
                return
            rank0 = self._round.by_rank.get(0)
            client = self._notify_clients.get((rank0.hostname, rank0.local_rank)) \
                if rank0 is not None else None
            if client is None:
                # kept for register_worker_server(): rank 0 is not listening yet
                self._undelivered_change |= change
                return
            self._undelivered_change = HostUpdateResult.no_update
        try:
            client.notify_hosts_updated(int(time.time()), change)
        except Exception:  # noqa: BLE001
            if self._verbose >= 2:
                logging.exception("could not notify rank 0 of the host change")
