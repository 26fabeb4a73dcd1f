"""Host discovery for elastic jobs: which hosts (and how many slots on each)
are available right now, what changed since the last look, and which hosts
are blacklisted after failures.

Parity: horovod/runner/elastic/discovery.py:80-186.
"""
import io
import threading
from collections import OrderedDict, defaultdict

from horovod_b200.common.elastic import HostUpdateResult
from horovod_b200.runner.common import safe_shell_exec


class HostState:
    def __init__(self):
        self._event = threading.Event()
        self._blacklisted = False

    def get_event(self):
        if self._event.is_set():
            self._event = threading.Event()
        return self._event

    def set_event(self):
        self._event.set()

    def blacklist(self):
        self._blacklisted = True
        self.set_event()

    def is_blacklisted(self):
        return self._blacklisted


class DiscoveredHosts:
    def __init__(self, host_slots, host_assignment_order):
        self._host_slots = dict(host_slots)
        self._host_assignment_order = list(host_assignment_order)

    @property
    def host_slots(self):
        return self._host_slots

    @property
    def available_hosts(self):
        return set(self._host_assignment_order)

    @property
    def host_assignment_order(self):
        return self._host_assignment_order

    def get_slots(self, host):
        return self._host_slots.get(host, 0)

    def count_available_slots(self):
        return sum(self.get_slots(h) for h in self._host_assignment_order)

    def update(self, hosts_state):
        self._host_assignment_order = [h for h in self._host_assignment_order
                                       if not hosts_state[h].is_blacklisted()]
        return self

    def __str__(self):
        return "slots: %s order: %s" % (self._host_slots, self._host_assignment_order)


class HostManager:
    def __init__(self, discovery):
        self._current_hosts = DiscoveredHosts(host_slots={}, host_assignment_order=[])
        self._hosts_state = defaultdict(HostState)
        self._discovery = discovery

    def update_available_hosts(self):
        """Polls discovery; returns a HostUpdateResult describing the change."""
        def check_update(cur_slots, prev_slots):
            res = HostUpdateResult.no_update
            for prev_h in prev_slots:
                if prev_h not in cur_slots:
                    res |= HostUpdateResult.removed
            for h, slots in cur_slots.items():
                if h not in prev_slots:
                    res |= HostUpdateResult.added
                elif slots > prev_slots[h]:
                    res |= HostUpdateResult.added
                elif slots < prev_slots[h]:
                    res |= HostUpdateResult.removed
            return res

        prev_slots = self._current_hosts.host_slots
        prev_order = self._current_hosts.host_assignment_order
        host_slots = self._discovery.find_available_hosts_and_slots()
        if prev_slots != host_slots:
            available = {h for h in host_slots if not self._hosts_state[h].is_blacklisted()}
            # Hosts that were already in use keep their place, so that an old
            # worker (which holds the training state) ends up as rank 0.
            order = [h for h in prev_order if h in available]
            order += [h for h in host_slots if h in available and h not in order]
            self._current_hosts = DiscoveredHosts(host_slots=host_slots,
                                                  host_assignment_order=order)
            return check_update(self._current_hosts.host_slots, prev_slots)
        return HostUpdateResult.no_update

    @property
    def current_hosts(self):
        return self._current_hosts.update(self._hosts_state)

    def blacklist(self, host):
        if not self._hosts_state[host].is_blacklisted():
            self._hosts_state[host].blacklist()

    def is_blacklisted(self, host):
        return self._hosts_state[host].is_blacklisted()

    def get_host_event(self, host):
        return self._hosts_state[host].get_event()


class HostDiscovery:
    def find_available_hosts_and_slots(self):
        """Returns an ordered dict hostname -> slots."""
        raise NotImplementedError()


class HostDiscoveryScript(HostDiscovery):
    """Runs a user script that prints one ``hostname[:slots]`` per line."""

    def __init__(self, discovery_script, slots):
        self._discovery_script = discovery_script
        self._default_slots = slots
        super().__init__()

    def find_available_hosts_and_slots(self):
        stdout = io.StringIO()
        exit_code = safe_shell_exec.execute(self._discovery_script, stdout=stdout)
        if exit_code != 0:
            raise RuntimeError("Failed to execute discovery script: %s. Exit code: %d"
                               % (self._discovery_script, exit_code))
        host_slots = OrderedDict()
        for line in set(stdout.getvalue().strip().split("\n")) - {""}:
            host = line.strip()
            if ":" in host:
                name, slots = host.rsplit(":", 1)
                host_slots[name] = int(slots)
            else:
                if self._default_slots is None:
                    raise ValueError("no slots given for host %s: pass --slots-per-host or "
                                     "print host:slots" % host)
                host_slots[host] = self._default_slots
        return OrderedDict(sorted(host_slots.items()))


class FixedHosts(HostDiscovery):
    def __init__(self, host_slots):
        super().__init__()
        self._host_slots = OrderedDict(host_slots)

    def find_available_hosts_and_slots(self):
        return self._host_slots

    def set(self, host_slots):
        self._host_slots = OrderedDict(host_slots)
