"""Host strings and slot assignment.

Parity: horovod/runner/common/util/hosts.py:33-155.
"""
import collections


class HostInfo:
    def __init__(self, hostname, slots):
        self.hostname = hostname
        self.slots = slots

    @staticmethod
    def from_string(host_string):
        hostname, _, slots = host_string.strip().partition(":")
        return HostInfo(hostname, int(slots) if slots else 1)

    def __repr__(self):
        return "%s:%d" % (self.hostname, self.slots)


class SlotInfo:
    """Place of one rank in the job."""

    def __init__(self, hostname, rank, local_rank, cross_rank, size, local_size, cross_size):
        self.hostname = hostname
        self.rank = rank
        self.local_rank = local_rank
        self.cross_rank = cross_rank
        self.size = size
        self.local_size = local_size
        self.cross_size = cross_size

    def to_response_string(self):
        return ",".join(str(v) for v in [self.rank, self.size, self.local_rank,
                                         self.local_size, self.cross_rank, self.cross_size])

    def __eq__(self, other):
        return isinstance(other, SlotInfo) and self.__dict__ == other.__dict__

    def __repr__(self):
        return "SlotInfo(%s)" % ", ".join("%s=%r" % kv for kv in sorted(self.__dict__.items()))


INVALID_SLOT_INFO = SlotInfo(hostname="", rank=-1, local_rank=-1, cross_rank=-1,
                             size=-1, local_size=-1, cross_size=-1)


def parse_hosts(hosts_string):
    """'h1:2,h2:4' -> [HostInfo]."""
    return [HostInfo.from_string(s) for s in hosts_string.split(",") if s.strip()]


def parse_hosts_and_slots(hosts_string):
    """'h1:2,h2:4' -> (['h1', 'h2'], {'h1': 2, 'h2': 4}); a host without a
    count has one slot."""
    parsed = parse_hosts(hosts_string)
    return [h.hostname for h in parsed], {h.hostname: h.slots for h in parsed}


def parse_host_files(filename):
    """Hostfile lines 'hostname slots=N' -> 'hostname:N,...'."""
    hosts = []
    with open(filename) as f:
        for line in f:
            line = line.strip()
            if not line or line.startswith("#"):
                continue
            parts = line.split()
            slots = 1
            for p in parts[1:]:
                if p.startswith("slots="):
                    slots = int(p[len("slots="):])
            hosts.append("%s:%d" % (parts[0], slots))
    return ",".join(hosts)


def get_host_assignments(hosts, min_np, max_np=None):
    """Fills hosts in order with consecutive ranks. Returns [SlotInfo] with
    at least min_np (else ValueError) and at most max_np entries."""
    host_ranks = []
    cross_ranks = collections.defaultdict(dict)
    rank = 0
    for host in hosts:
        ranks = []
        for local_rank in range(host.slots):
            if rank == max_np:
                break
            ranks.append(rank)
            rank += 1
            cross_ranks_at_local = cross_ranks[local_rank]
            cross_ranks_at_local[host.hostname] = len(cross_ranks_at_local)
        host_ranks.append((host, ranks))
    world_size = rank
    if world_size < min_np:
        raise ValueError("Requested more processes (%d) than there are available slots (%d)"
                         % (min_np, world_size))
    alloc = []
    for host, ranks in host_ranks:
        local_size = len(ranks)
        for local_rank, r in enumerate(ranks):
            at_local = cross_ranks[local_rank]
            alloc.append(SlotInfo(hostname=host.hostname, rank=r, local_rank=local_rank,
                                  cross_rank=at_local[host.hostname], size=world_size,
                                  local_size=local_size, cross_size=len(at_local)))
    return alloc


def host_hash(salt=None):
    """Identifies "the same machine" for slot grouping: two processes that
    share a hostname (and salt) share a host. Parity:
    horovod/runner/common/util/host_hash.py:21-48."""
    import hashlib
    import socket
    name = socket.gethostname().split(".")[0]
    if salt is not None:
        name = "%s-%s" % (name, salt)
    return "%s-%s" % (name, hashlib.md5(name.encode("ascii", "ignore")).hexdigest())
