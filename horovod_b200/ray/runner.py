"""Ray integration: one actor per rank, a coordinator that turns the actors'
(host, node, rank) registrations into per-rank environments and starts the
rendezvous server, and an executor with start / run / execute / shutdown.
``ray`` is imported only when an executor is started, so everything else here
(the coordinator's arithmetic) works and is tested without it.
Parity: horovod/ray/runner.py:41-126 (Coordinator), :128-430 (RayExecutor).
"""
import collections
import os
import socket

from horovod_b200.runner.common import hosts as hosts_mod
from horovod_b200.runner.http.http_server import RendezvousServer, local_ip_for


def _require_ray():
    try:
        import ray
        return ray
    except ImportError as e:  # pragma: no cover - depends on the environment
        raise ImportError("horovod_b200.ray needs the `ray` package, which is not "
                          "installed in this environment.") from e


class Coordinator:
    """Collects ``register(hostname, node_id, world_rank)`` calls and derives
    every rank's local/cross coordinates: ranks on one node get consecutive
    local ranks in registration order; the cross rank of a rank is the index
    of its node among the nodes that have that local rank."""

    def __init__(self, settings=None):
        self.settings = settings
        self._ranks_by_node = collections.OrderedDict()
        self._hostnames = set()
        self.rendezvous = None
        self.global_rendezv_port = None

    @property
    def world_size(self):
        return sum(len(r) for r in self._ranks_by_node.values())

    @property
    def hostnames(self):
        return set(self._hostnames)

    @property
    def node_id_string(self):
        return ",".join("%s:%d" % (node, len(ranks))
                        for node, ranks in self._ranks_by_node.items())

    def register(self, hostname, node_id, world_rank):
        self._hostnames.add(hostname)
        self._ranks_by_node.setdefault(node_id, []).append(world_rank)

    def finalize_registration(self):
        """{world_rank: {HOROVOD_* coordinates}} for all registered ranks."""
        nodes_with_local = collections.defaultdict(int)
        cross_rank = {}
        for ranks in self._ranks_by_node.values():
            for local_rank, world_rank in enumerate(ranks):
                cross_rank[world_rank] = nodes_with_local[local_rank]
                nodes_with_local[local_rank] += 1
        info = {}
        size = self.world_size
        for ranks in self._ranks_by_node.values():
            for local_rank, world_rank in enumerate(ranks):
                info[world_rank] = {
                    "HOROVOD_RANK": world_rank,
                    "HOROVOD_SIZE": size,
                    "HOROVOD_LOCAL_RANK": local_rank,
                    "HOROVOD_LOCAL_SIZE": len(ranks),
                    "HOROVOD_CROSS_RANK": cross_rank[world_rank],
                    "HOROVOD_CROSS_SIZE": nodes_with_local[local_rank],
                }
        return info

    def establish_rendezvous(self, advertise_ip=None):
        """Starts the rendezvous server for the registered layout and returns
        the environment every worker needs to find it."""
        self.rendezvous = RendezvousServer(getattr(self.settings, "verbose", 0) or 0)
        parsed = hosts_mod.parse_hosts(self.node_id_string)
        plan = hosts_mod.get_host_assignments(parsed, self.world_size)
        self.global_rendezv_port = self.rendezvous.start()
        self.rendezvous.init(plan)
        return {
            "HOROVOD_GLOO_RENDEZVOUS_ADDR": advertise_ip or local_ip_for(),
            "HOROVOD_GLOO_RENDEZVOUS_PORT": str(self.global_rendezv_port),
            "HOROVOD_CONTROLLER": "gloo",
            "HOROVOD_CPU_OPERATIONS": "gloo",
        }

    def shutdown(self):
        if self.rendezvous is not None:
            self.rendezvous.stop()
            self.rendezvous = None


class _Worker:
    """Body of the Ray actor of one rank."""

    def __init__(self, world_rank):
        self.world_rank = world_rank
        self.executable = None

    def hostname(self):
        return socket.gethostname()

    def node_id(self):
        ray = _require_ray()
        return ray.get_runtime_context().get_node_id()

    def update_env_vars(self, env):
        os.environ.update({k: str(v) for k, v in env.items()})

    def env_vars(self):
        return dict(os.environ)

    def start_executable(self, executable_cls=None, executable_args=None,
                         executable_kwargs=None):
        if executable_cls is not None:
            self.executable = executable_cls(*(executable_args or []),
                                             **(executable_kwargs or {}))

    def execute(self, fn):
        return fn(self.executable)

    def run(self, fn, args, kwargs):
        return fn(*args, **kwargs)


class RayExecutor:
    """``RayExecutor(settings, num_workers=8, use_gpu=True).start()`` creates
    the actors and the rendezvous; ``run(fn, args)`` runs ``fn`` on every rank
    (``hvd.init()`` inside works as under the launcher) and returns the
    results by rank; ``execute(fn)`` calls ``fn(executable)`` on the optional
    per-rank object; ``shutdown()`` kills the actors."""

    @classmethod
    def create_settings(cls, timeout_s=30, ssh_identity_file=None, ssh_str=None,
                        placement_group_timeout_s=100, nics=None):
        from horovod_b200.runner.common.settings import Settings
        from horovod_b200.runner.common.timeout import Timeout
        return Settings(verbose=1, ssh_identity_file=ssh_identity_file, nics=nics,
                        start_timeout=Timeout(timeout_s, "Timed out waiting for {activity}."))

    def __init__(self, settings=None, num_workers=None, num_hosts=None,
                 num_workers_per_host=1, cpus_per_worker=1, use_gpu=False,
                 gpus_per_worker=None, use_placement_group=True,
                 placement_group_timeout_s=100):
        if num_workers is None and num_hosts is None:
            raise ValueError("Either `num_workers` or `num_hosts` must be specified.")
        if num_workers is not None and num_hosts is not None:
            raise ValueError("Specify `num_workers` or `num_hosts` (with "
                             "`num_workers_per_host`), not both.")
        if gpus_per_worker and not use_gpu:
            raise ValueError("gpus_per_worker is set, but use_gpu is False.")
        self.settings = settings
        self.num_workers = num_workers if num_workers is not None \
            else num_hosts * num_workers_per_host
        self.cpus_per_worker = cpus_per_worker
        self.use_gpu = use_gpu
        self.gpus_per_worker = gpus_per_worker or (1 if use_gpu else 0)
        self.workers = []
        self.coordinator = None
        # Where the actors go (horovod/ray/strategy.py): packed, or a fixed
        # number per host with every host on its own node.
        from horovod_b200.ray import strategy
        if num_workers is not None:
            self.plan = strategy.plan_packed(self.num_workers, cpus_per_worker,
                                             self.gpus_per_worker)
        else:
            self.plan = strategy.plan_colocated(num_hosts, num_workers_per_host,
                                                cpus_per_worker, self.gpus_per_worker)
        self.use_placement_group = use_placement_group
        self.placement_group_timeout_s = placement_group_timeout_s
        self.placement = None

    def start(self, executable_cls=None, executable_args=None, executable_kwargs=None,
              extra_env_vars=None):
        ray = _require_ray()
        from horovod_b200.ray.strategy import PlacementGroupHandle
        self.placement = PlacementGroupHandle(ray, self.plan)
        if self.use_placement_group:
            self.placement.create(self.placement_group_timeout_s)
        remote_cls = ray.remote(_Worker)
        self.workers = [remote_cls.options(**self.placement.actor_options(r)).remote(world_rank=r)
                        for r in range(self.num_workers)]
        hostnames = ray.get([w.hostname.remote() for w in self.workers])
        node_ids = ray.get([w.node_id.remote() for w in self.workers])
        self.coordinator = Coordinator(self.settings)
        for rank, (hostname, node_id) in enumerate(zip(hostnames, node_ids)):
            self.coordinator.register(hostname, node_id, rank)
        per_rank = self.coordinator.finalize_registration()
        common = self.coordinator.establish_rendezvous(ray.util.get_node_ip_address())
        common.update(extra_env_vars or {})
        ray.get([w.update_env_vars.remote(dict(common, **per_rank[r]))
                 for r, w in enumerate(self.workers)])
        ray.get([w.start_executable.remote(executable_cls, executable_args, executable_kwargs)
                 for w in self.workers])

    def run(self, fn, args=None, kwargs=None):
        ray = _require_ray()
        return ray.get(self.run_remote(fn, args, kwargs))

    def run_remote(self, fn, args=None, kwargs=None):
        return [w.run.remote(fn, args or [], kwargs or {}) for w in self.workers]

    def execute(self, fn):
        ray = _require_ray()
        return ray.get([w.execute.remote(fn) for w in self.workers])

    def execute_single(self, fn):
        ray = _require_ray()
        return ray.get(self.workers[0].execute.remote(fn))

    def shutdown(self):
        ray = _require_ray()
        for w in self.workers:
            ray.kill(w)
        self.workers = []
        if self.placement is not None:
            self.placement.remove()
            self.placement = None
        if self.coordinator is not None:
            self.coordinator.shutdown()
            self.coordinator = None
