"""Running a job on a Ray cluster (needs the ``ray`` package at call time)."""
from horovod_b200.ray.runner import Coordinator, RayExecutor  # noqa: F401
from horovod_b200.ray.elastic import ElasticRayExecutor, RayHostDiscovery  # noqa: F401
from horovod_b200.ray.strategy import plan_colocated, plan_packed  # noqa: F401
