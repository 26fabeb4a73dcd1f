"""Process sets: named subsets of ranks that run collectives among themselves.

``global_process_set`` (id 0) always exists. Further sets are either passed
to ``hvd.init(process_sets=[...])`` or, when the job runs with
``HOROVOD_DYNAMIC_PROCESS_SETS=1`` / ``init(process_sets="dynamic")``, added
and removed at run time by calling add_process_set / remove_process_set with
the same arguments on every rank.

Parity: horovod/common/process_sets.py:18-163. Unlike that snapshot, every
PyTorch collective here accepts ``process_set=``.
"""


def _native():
    from horovod_b200 import _C
    return _C


class ProcessSet:
    """A set of global ranks. ``process_set_id`` is filled in once the set is
    registered with the runtime."""

    def __init__(self, ranks_or_comm):
        self.process_set_id = None
        self.ranks = sorted(set(int(r) for r in ranks_or_comm))

    def _invalidate(self):
        self.process_set_id = None

    def size(self):
        """Number of ranks in the set (None before registration)."""
        if self.process_set_id is None:
            return None
        return _native().process_set_size(self.process_set_id)

    def rank(self):
        """This process's rank inside the set, or -1 if it is not a member."""
        if self.process_set_id is None:
            return None
        return _native().process_set_rank(self.process_set_id)

    def included(self):
        if self.process_set_id is None:
            return None
        return _native().process_set_included(self.process_set_id)

    def __str__(self):
        return "ProcessSet(process_set_id=%s, ranks=%s)" % (self.process_set_id, self.ranks)

    __repr__ = __str__


global_process_set = ProcessSet([])
global_process_set.process_set_id = 0

_registered = {}  # id -> ProcessSet object handed to the user


def _init_process_sets(process_sets):
    """Binds ids to the objects passed to init() and refreshes the global set."""
    _C = _native()
    global_process_set.ranks = list(range(_C.size()))
    global_process_set.process_set_id = 0
    for obj in list(_registered.values()):
        if obj is not global_process_set:
            obj._invalidate()
    _registered.clear()
    _registered[0] = global_process_set
    id_by_ranks = {tuple(_C.process_set_ranks(i)): i for i in _C.process_set_ids()}
    for ps in process_sets:
        if not isinstance(ps, ProcessSet):
            continue
        ps.process_set_id = id_by_ranks.get(tuple(ps.ranks))
        if ps.process_set_id is not None:
            _registered[ps.process_set_id] = ps


def add_process_set(process_set):
    """Registers a new set on all ranks (collective call). Accepts a
    ProcessSet or a list of ranks; returns the ProcessSet with its id."""
    if not isinstance(process_set, ProcessSet):
        process_set = ProcessSet(process_set)
    _C = _native()
    try:
        pid = _C.add_process_set(process_set.ranks)
    except RuntimeError as e:
        raise ValueError(str(e))
    if pid in _registered and _registered[pid] is not process_set:
        raise ValueError("A process set with ranks %s already exists." % process_set.ranks)
    process_set.process_set_id = pid
    _registered[pid] = process_set
    return process_set


def remove_process_set(process_set):
    """Removes a set on all ranks (collective call). Returns True if it was
    registered. The global set cannot be removed."""
    pid = process_set.process_set_id
    if pid is None or pid == 0:
        return False
    _C = _native()
    try:
        _C.remove_process_set(pid)
    except RuntimeError as e:
        raise ValueError(str(e))
    _registered.pop(pid, None)
    process_set._invalidate()
    return True


def process_set_ids():
    return list(_native().process_set_ids())


def _resolve(process_set):
    """Maps the process_set= argument of an op to a registered id."""
    if process_set is None:
        return 0
    if isinstance(process_set, int):
        return process_set
    if process_set.process_set_id is None:
        raise ValueError("%s has not been registered; pass it to hvd.init() or "
                         "hvd.add_process_set()." % process_set)
    return process_set.process_set_id
