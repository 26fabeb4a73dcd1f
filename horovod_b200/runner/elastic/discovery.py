"""Host discovery for elastic jobs.

A ``HostDiscovery`` answers "which hosts, with how many slots each, could run
workers right now". ``HostManager`` polls one, remembers since when each host
has been around (hosts that have been in the job longest come first when ranks
are handed out, so that a worker which already holds training state becomes
rank 0), reports what changed between two polls, and keeps the list of hosts
that must not be used again after a failure.

Behaviour follows horovod/runner/elastic/discovery.py:80-186 (script output
format ``host[:slots]``, add/remove classification, blacklist, survivor-first
ordering); the bookkeeping here is a seniority table instead of ordered host
lists.
"""
import io
import itertools
import threading
from collections import OrderedDict

from horovod_b200.common.elastic import HostUpdateResult
from horovod_b200.runner.common import safe_shell_exec


class HostDiscovery:
    def find_available_hosts_and_slots(self):
        """Returns an ordered mapping hostname -> slots."""
        raise NotImplementedError()


class HostDiscoveryScript(HostDiscovery):
    """Runs a user script that prints one ``hostname[:slots]`` per line; hosts
    without a slot count get ``slots`` (the --slots-per-host value)."""

    def __init__(self, discovery_script, slots):
        self._script = discovery_script
        self._slots_per_host = slots

    def find_available_hosts_and_slots(self):
        out = io.StringIO()
        code = safe_shell_exec.execute(self._script, stdout=out)
        if code != 0:
            raise RuntimeError("Failed to execute discovery script: %s. Exit code: %d"
                               % (self._script, code))
        found = {}
        for raw in out.getvalue().splitlines():
            entry = raw.strip()
            if not entry:
                continue
            name, sep, count = entry.rpartition(":")
            if sep:
                found[name] = int(count)
            elif self._slots_per_host is not None:
                found[entry] = self._slots_per_host
            else:
                raise ValueError("no slots given for host %s: pass --slots-per-host or "
                                 "print host:slots" % entry)
        return OrderedDict((h, found[h]) for h in sorted(found))


class FixedHosts(HostDiscovery):
    """A host list that only changes when ``set`` is called (tests, static
    host lists run through the elastic driver)."""

    def __init__(self, host_slots):
        self._host_slots = OrderedDict(host_slots)

    def find_available_hosts_and_slots(self):
        return self._host_slots

    def set(self, host_slots):
        self._host_slots = OrderedDict(host_slots)


class HostView:
    """What the manager knew at one moment: every discovered host with its
    slots, and the usable (not blacklisted) ones in rank-assignment order."""

    def __init__(self, host_slots, usable_in_order):
        self.host_slots = dict(host_slots)
        self.host_assignment_order = list(usable_in_order)

    @property
    def available_hosts(self):
        return set(self.host_assignment_order)

    def get_slots(self, host):
        return self.host_slots.get(host, 0)

    def count_available_slots(self):
        return sum(self.host_slots[h] for h in self.host_assignment_order)

    def __repr__(self):
        return "HostView(slots=%r, order=%r)" % (self.host_slots, self.host_assignment_order)


class HostManager:
    def __init__(self, discovery):
        self._discovery = discovery
        self._lock = threading.Lock()
        self._slots = OrderedDict()     # host -> slots, as last discovered
        self._seniority = {}            # host -> ticket; lower = longer in the job
        self._tickets = itertools.count()
        self._banned = set()
        self._ban_events = {}           # host -> Event set when the host is banned

    def update_available_hosts(self):
        """Polls discovery once and classifies the change against the previous
        poll: a host that gained slots (or appeared) counts as ``added``, one
        that lost slots (or vanished) as ``removed``; both at once is
        ``mixed``."""
        latest = OrderedDict(self._discovery.find_available_hosts_and_slots())
        with self._lock:
            change = HostUpdateResult.no_update
            for host in set(self._slots) | set(latest):
                before, after = self._slots.get(host, 0), latest.get(host, 0)
                if after > before:
                    change |= HostUpdateResult.added
                elif after < before:
                    change |= HostUpdateResult.removed
            # A host that left and later returns queues up behind the others.
            for host in list(self._seniority):
                if host not in latest:
                    del self._seniority[host]
            for host in latest:
                if host not in self._seniority:
                    self._seniority[host] = next(self._tickets)
            self._slots = latest
            return change

    @property
    def current_hosts(self):
        with self._lock:
            usable = [h for h in self._slots if h not in self._banned]
            usable.sort(key=self._seniority.__getitem__)
            return HostView(self._slots, usable)

    def blacklist(self, host):
        with self._lock:
            if host in self._banned:
                return
            self._banned.add(host)
            event = self._ban_events.get(host)
        if event is not None:
            event.set()

    def is_blacklisted(self, host):
        with self._lock:
            return host in self._banned

    def get_host_event(self, host):
        """An event that fires when ``host`` is blacklisted (the launcher uses
        it to terminate the host's worker processes)."""
        with self._lock:
            event = self._ban_events.get(host)
            if event is None or (event.is_set() and host not in self._banned):
                event = self._ban_events[host] = threading.Event()
            if host in self._banned:
                event.set()
            return event
