"""Exception types raised by the framework.

Parity: horovod/common/exceptions.py:18-49.
"""


class HorovodInternalError(RuntimeError):
    """A collective failed for a reason outside the caller's control (a peer
    died, the runtime shut down). Elastic training catches it, restores the
    last committed state and re-initialises."""


class WorkerRemovedError(HorovodInternalError):
    """The elastic driver no longer has a place for this worker (its host
    left the job). Raised by ``init()`` after a reset; the elastic retry loop
    ends the process quietly with exit code 0 when it sees it."""


class HostsUpdatedInterrupt(RuntimeError):
    """The set of hosts changed; raised at a commit point so every rank can
    re-rendezvous. ``skip_sync`` is true when only removals happened, in which
    case the surviving ranks already hold identical state."""

    def __init__(self, skip_sync):
        super().__init__()
        self.skip_sync = skip_sync


class HorovodVersionMismatchError(ImportError):
    """The installed native module was built for another framework version."""

    def __init__(self, name, version, installed_version):
        super().__init__(
            "Framework %s installed with version %s but found version %s. "
            "Rebuild the native module (python horovod_b200/build_ext.py)."
            % (name, installed_version, version))
        self.name = name
        self.version = version
        self.installed_version = installed_version


def get_version_mismatch_message(name, version, installed_version):
    return str(HorovodVersionMismatchError(name, version, installed_version))
