"""Lifecycle and topology queries: init / shutdown / rank / size and friends.

``init()`` works out this process's place in the job from the environment,
exchanges the address of its control socket with the other ranks through
whichever rendezvous the launcher offers, and starts the native runtime.
Three launch styles are understood:

* ``horovodrun`` (this package's launcher): ``HOROVOD_RANK/SIZE/LOCAL_RANK/...``
  plus an HTTP key-value rendezvous at ``HOROVOD_GLOO_RENDEZVOUS_ADDR:PORT``.
* ``torchrun``: ``RANK/WORLD_SIZE/LOCAL_RANK/MASTER_ADDR/MASTER_PORT`` with a
  ``torch.distributed.TCPStore`` as the key-value store.
* nothing set: a single-process job.

Parity: horovod/common/basics.py:29-487 and the rendezvous half of
horovod/common/gloo/gloo_context.cc:134-232 (including the elastic re-query
of rank and size, :168-214).
"""
import atexit
import os
import socket
import time
import urllib.error
import urllib.request

from horovod_b200.common.exceptions import HorovodInternalError, WorkerRemovedError

_GENERATION = [0]
_TORCH_STORE = [None]


def _native():
    from horovod_b200 import _C
    return _C


class _HttpKV:
    """Client of the launcher's rendezvous server."""

    def __init__(self, addr, port):
        self.base = "http://%s:%d" % (addr, int(port))

    def put(self, scope, key, value):
        data = value if isinstance(value, bytes) else str(value).encode()
        deadline = time.time() + 60
        while True:
            try:
                req = urllib.request.Request("%s/%s/%s" % (self.base, scope, key),
                                             data=data, method="PUT")
                with urllib.request.urlopen(req, timeout=30):
                    return
            except (urllib.error.URLError, OSError):
                if time.time() > deadline:
                    raise
                time.sleep(0.05)

    def get(self, scope, key, timeout=300.0):
        deadline = time.time() + timeout
        while True:
            try:
                url = "%s/%s/%s" % (self.base, scope, key)
                with urllib.request.urlopen(url, timeout=max(1.0, deadline - time.time())) as r:
                    return r.read()
            except urllib.error.HTTPError as e:
                if e.code != 404:
                    raise
            except (urllib.error.URLError, OSError):
                pass
            if time.time() > deadline:
                raise TimeoutError("rendezvous key %s/%s never appeared" % (scope, key))
            time.sleep(0.01)

    def delete(self, scope, key):
        try:
            req = urllib.request.Request("%s/%s/%s" % (self.base, scope, key),
                                         method="DELETE")
            with urllib.request.urlopen(req, timeout=5):
                pass
        except (urllib.error.URLError, OSError):
            pass


def _route_ip(addr, port):
    """The local address a peer on the rendezvous server's network can reach:
    the source address of a connection towards that server."""
    override = os.environ.get("HOROVOD_ADVERTISE_ADDR")
    if override:
        return override
    if addr in ("127.0.0.1", "localhost", "::1"):
        return "127.0.0.1"
    try:
        s = socket.create_connection((addr, int(port)), timeout=5)
        ip = s.getsockname()[0]
        s.close()
        return ip
    except OSError:
        return "127.0.0.1"


def _layout_from_env():
    """Returns (layout dict, kv exchange function) or (None, None) for a
    single-process job."""
    env = os.environ
    if "HOROVOD_RANK" in env and "HOROVOD_SIZE" in env:
        addr = env.get("HOROVOD_GLOO_RENDEZVOUS_ADDR")
        port = env.get("HOROVOD_GLOO_RENDEZVOUS_PORT")
        layout = dict(
            rank=int(env["HOROVOD_RANK"]), size=int(env["HOROVOD_SIZE"]),
            local_rank=int(env.get("HOROVOD_LOCAL_RANK", 0)),
            local_size=int(env.get("HOROVOD_LOCAL_SIZE", 1)),
            cross_rank=int(env.get("HOROVOD_CROSS_RANK", 0)),
            cross_size=int(env.get("HOROVOD_CROSS_SIZE", 1)))
        if layout["size"] == 1 and not addr:
            return layout, None
        if not addr or not port:
            raise RuntimeError("HOROVOD_RANK/SIZE are set but the rendezvous "
                               "address HOROVOD_GLOO_RENDEZVOUS_ADDR/PORT is not.")
        kv = _HttpKV(addr, port)
        if env.get("HOROVOD_ELASTIC") == "1" and _GENERATION[0] > 0:
            # Re-initialisation inside an elastic job: ask the driver for this
            # worker's new place. The request blocks until every worker that
            # survived the previous round has asked. (A freshly spawned worker
            # instead uses the layout and round number it was started with.)
            host = env.get("HOROVOD_HOSTNAME", socket.gethostname())
            key = "%s:%s" % (host, env.get("HOROVOD_LOCAL_RANK", "0"))
            timeout = float(env.get("HOROVOD_ELASTIC_TIMEOUT", "600"))
            reply = kv.get("rank_and_size", key, timeout=timeout).decode()
            vals = [int(v) for v in reply.split(",")]
            if vals[0] < 0:
                raise WorkerRemovedError(
                    "This worker was removed from the job by the elastic driver.")
            names = ["rank", "size", "local_rank", "local_size", "cross_rank", "cross_size"]
            layout = dict(zip(names, vals[:6]))
            for n in names:
                os.environ["HOROVOD_" + n.upper()] = str(layout[n])
            scope = "global_%d" % (vals[6] if len(vals) > 6 else 0)
        elif env.get("HOROVOD_ELASTIC") == "1":
            scope = "global_%s" % env.get("HOROVOD_ELASTIC_ROUND", "0")
        else:
            scope = "global"
        advertise = _route_ip(addr, port)

        def exchange(my_addr):
            kv.put(scope, "addr_%d" % layout["rank"], my_addr)
            addrs = [kv.get(scope, "addr_%d" % r).decode() for r in range(layout["size"])]
            token = int.from_bytes(
                __import__("hashlib").sha256((scope + addrs[0]).encode()).digest()[:8], "little")
            return addrs, token

        return dict(layout, advertise=advertise), exchange

    if "RANK" in env and "WORLD_SIZE" in env and int(env["WORLD_SIZE"]) > 1:
        rank, size = int(env["RANK"]), int(env["WORLD_SIZE"])
        local_rank = int(env.get("LOCAL_RANK", rank))
        local_size = int(env.get("LOCAL_WORLD_SIZE", size))
        layout = dict(rank=rank, size=size, local_rank=local_rank,
                      local_size=local_size,
                      cross_rank=int(env.get("GROUP_RANK", rank // max(1, local_size))),
                      cross_size=max(1, size // max(1, local_size)))
        addr, port = env.get("MASTER_ADDR", "127.0.0.1"), int(env.get("MASTER_PORT", "29500"))
        advertise = _route_ip(addr, port)

        def exchange(my_addr):
            from datetime import timedelta
            import torch.distributed as dist
            if _TORCH_STORE[0] is None:
                agent = env.get("TORCHELASTIC_USE_AGENT_STORE", "False") == "True"
                _TORCH_STORE[0] = dist.TCPStore(
                    addr, port, size, is_master=(rank == 0 and not agent),
                    timeout=timedelta(seconds=300), wait_for_workers=False)
            store = _TORCH_STORE[0]
            gen = _GENERATION[0]
            store.set("hvdb200/%d/addr/%d" % (gen, rank), my_addr)
            addrs = [store.get("hvdb200/%d/addr/%d" % (gen, r)).decode() for r in range(size)]
            token = int.from_bytes(
                __import__("hashlib").sha256(("%d" % gen + addrs[0]).encode()).digest()[:8], "little")
            return addrs, token

        return dict(layout, advertise=advertise), exchange

    return None, None


class HorovodBasics:
    """Process-wide lifecycle and topology API (one instance per binding)."""

    def __init__(self):
        self._atexit_registered = False

    def init(self, comm=None, process_sets=None):
        """Starts the runtime. ``comm`` may be a list of ranks (kept for API
        compatibility; ranks outside the list are not supported in this
        single-world design and raise). ``process_sets`` is a list of
        ``ProcessSet`` objects or rank lists to register at start-up, or the
        string "dynamic" to allow add_process_set()/remove_process_set()
        afterwards."""
        from horovod_b200.common import process_sets as ps_mod
        _C = _native()
        if _C.is_initialized():
            return
        if comm is not None and not isinstance(comm, (list, tuple)):
            raise ValueError("init(comm=...) accepts only a list of ranks here; "
                             "MPI communicators are not supported.")
        if isinstance(process_sets, str):
            if process_sets.lower() != "dynamic":
                raise ValueError("process_sets must be a list or 'dynamic'")
            os.environ["HOROVOD_DYNAMIC_PROCESS_SETS"] = "1"
            process_sets = []
        process_sets = list(process_sets or [])
        rank_lists = []
        for ps in process_sets:
            ranks = ps.ranks if isinstance(ps, ps_mod.ProcessSet) else list(ps)
            rank_lists.append(sorted(set(int(r) for r in ranks)))

        layout, exchange = _layout_from_env()
        _GENERATION[0] += 1
        if layout is None or exchange is None:
            lay = layout or dict(rank=0, size=1, local_rank=0, local_size=1,
                                 cross_rank=0, cross_size=1)
            _C.init(lay["rank"], 1, lay["local_rank"], 1, 0, 1, [], 0, rank_lists)
        else:
            my_addr = _C.listen(layout["advertise"])
            addrs, token = exchange(my_addr)
            try:
                _C.init(layout["rank"], layout["size"], layout["local_rank"],
                        layout["local_size"], layout["cross_rank"],
                        layout["cross_size"], addrs, token, rank_lists)
            except RuntimeError as e:
                raise HorovodInternalError(str(e))
        if comm is not None and sorted(comm) != list(range(_C.size())):
            _C.shutdown()
            raise ValueError("init(comm=[...]) must list every rank of the job; "
                             "use process sets for sub-groups.")
        ps_mod._init_process_sets(process_sets)
        if not self._atexit_registered:
            atexit.register(self.shutdown)
            self._atexit_registered = True

    def shutdown(self):
        """Stops the background thread on every rank and releases sockets and
        device buffers. ``init()`` may be called again afterwards."""
        _C = _native()
        _C.shutdown()

    def is_initialized(self):
        return _native().is_initialized()

    def _check(self):
        # rank()/size() stay answerable after a peer has shut the job down
        # (collectives then fail with HorovodInternalError instead).
        if not _native().has_topology():
            raise ValueError("Horovod has not been initialized; use hvd.init().")

    def size(self):
        self._check()
        return _native().size()

    def rank(self):
        self._check()
        return _native().rank()

    def local_size(self):
        self._check()
        return _native().local_size()

    def local_rank(self):
        self._check()
        return _native().local_rank()

    def cross_size(self):
        self._check()
        return _native().cross_size()

    def cross_rank(self):
        self._check()
        return _native().cross_rank()

    def is_homogeneous(self):
        self._check()
        return _native().is_homogeneous()

    def start_timeline(self, file_path, mark_cycles=False):
        """Starts writing the Chrome-trace timeline to ``file_path`` (rank 0
        writes; other ranks ignore the call)."""
        self._check()
        _native().start_timeline(str(file_path), bool(mark_cycles))

    def stop_timeline(self):
        self._check()
        _native().stop_timeline()

    # Build-feature queries kept for scripts that branch on them. This
    # framework has exactly one configuration.
    def mpi_threads_supported(self):
        return False

    def mpi_enabled(self):
        return False

    def mpi_built(self):
        return False

    def gloo_enabled(self):
        return True

    def gloo_built(self):
        return True

    def nccl_built(self):
        return 1

    def ddl_built(self):
        return False

    def ccl_built(self):
        return False

    def cuda_built(self):
        return True

    def rocm_built(self):
        return False

    def topology(self):
        """What the GPUs of this box look like: peer access / P2P attributes
        between every pair, active NVLink links, NVLink multicast support
        (dict; device_count is 0 without a GPU)."""
        return _native().gpu_topology()

    def gpu_backend(self):
        """Which device data path is active: "symm ..." (NVLink kernels over
        symmetric memory), "nccl" or "none"."""
        return _native().gpu_backend()

    def runtime_params(self):
        """The tunables as they are in effect now (the autotuner may have moved
        them): fusion_threshold_bytes, cycle_time_ms, cache_enabled,
        hierarchical_allreduce, hierarchical_allgather, autotune."""
        return dict(_native().runtime_params())
