"""Where the actors of a RayExecutor go: a placement plan (bundles of CPU/GPU
resources and a Ray placement strategy) computed from the executor's
arguments, and the placement group built from it.

Two layouts, as in horovod/ray/strategy.py:62-204:
  * ``num_workers``: one bundle per worker, packed onto as few nodes as
    possible (Ray strategy "PACK"); ranks end up wherever Ray has room.
  * ``num_hosts`` x ``num_workers_per_host``: one bundle per host that holds the
    resources of all its workers, every bundle on a different node
    ("STRICT_SPREAD"); rank r runs in bundle r // num_workers_per_host.
The plan itself is plain data, so it is tested without Ray.
"""


class PlacementPlan:
    """bundles: list of resource dicts; strategy: Ray placement strategy name;
    bundle_of_rank: which bundle each rank's actor is scheduled into."""

    def __init__(self, bundles, strategy, bundle_of_rank, cpus_per_worker, gpus_per_worker):
        self.bundles = bundles
        self.strategy = strategy
        self.bundle_of_rank = bundle_of_rank
        self.cpus_per_worker = cpus_per_worker
        self.gpus_per_worker = gpus_per_worker

    @property
    def num_workers(self):
        return len(self.bundle_of_rank)


def _resources(cpus, gpus):
    res = {"CPU": cpus}
    if gpus:
        res["GPU"] = gpus
    return res


def plan_packed(num_workers, cpus_per_worker=1, gpus_per_worker=0):
    if num_workers < 1:
        raise ValueError("num_workers must be positive")
    bundles = [_resources(cpus_per_worker, gpus_per_worker) for _ in range(num_workers)]
    return PlacementPlan(bundles, "PACK", list(range(num_workers)), cpus_per_worker,
                         gpus_per_worker)


def plan_colocated(num_hosts, num_workers_per_host, cpus_per_worker=1, gpus_per_worker=0):
    if num_hosts < 1 or num_workers_per_host < 1:
        raise ValueError("num_hosts and num_workers_per_host must be positive")
    per_host = _resources(cpus_per_worker * num_workers_per_host,
                          gpus_per_worker * num_workers_per_host)
    bundles = [dict(per_host) for _ in range(num_hosts)]
    ranks = [r // num_workers_per_host for r in range(num_hosts * num_workers_per_host)]
    return PlacementPlan(bundles, "STRICT_SPREAD", ranks, cpus_per_worker, gpus_per_worker)


class PlacementGroupHandle:
    """The Ray placement group of a plan. ``create`` waits until Ray has
    reserved every bundle (or raises TimeoutError and removes the group);
    ``actor_options(rank)`` are the options that schedule rank's actor into
    its bundle."""

    def __init__(self, ray, plan):
        self.ray = ray
        self.plan = plan
        self.group = None

    def create(self, timeout_s=100):
        from ray.util import placement_group
        self.group = placement_group(self.plan.bundles, strategy=self.plan.strategy)
        ready, _ = self.ray.wait([self.group.ready()], timeout=timeout_s)
        if not ready:
            self.remove()
            raise TimeoutError(
                "Ray could not reserve %d bundle(s) %s within %d s; the cluster has %s."
                % (len(self.plan.bundles), self.plan.bundles[0], timeout_s,
                   self.ray.available_resources()))
        return self

    def actor_options(self, rank):
        opts = {"num_cpus": self.plan.cpus_per_worker, "num_gpus": self.plan.gpus_per_worker}
        if self.group is not None:
            opts["placement_group"] = self.group
            opts["placement_group_bundle_index"] = self.plan.bundle_of_rank[rank]
        return opts

    def remove(self):
        if self.group is not None:
            from ray.util import remove_placement_group
            remove_placement_group(self.group)
            self.group = None
