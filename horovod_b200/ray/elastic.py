"""Host discovery for elastic jobs on Ray: the alive nodes of the cluster and
how many slots each can host, from their CPU/GPU resources.
Parity: horovod/ray/elastic.py:38-94 (RayHostDiscovery)."""
from horovod_b200.runner.elastic.discovery import HostDiscovery


class RayHostDiscovery(HostDiscovery):
    def __init__(self, use_gpu=False, cpus_per_slot=1, gpus_per_slot=1):
        self.use_gpu = use_gpu
        self.cpus_per_slot = cpus_per_slot
        self.gpus_per_slot = gpus_per_slot

    def find_available_hosts_and_slots(self):
        """{node address: slots} over the alive nodes of the Ray cluster."""
        from horovod_b200.ray.runner import _require_ray
        ray = _require_ray()
        mapping = {}
        for node in ray.nodes():
            if not node.get("alive", node.get("Alive", False)):
                continue
            resources = node.get("Resources", {})
            hostname = node.get("NodeManagerAddress")
            slots = resources.get("CPU", 0) // self.cpus_per_slot
            if self.use_gpu:
                slots = min(slots, resources.get("GPU", 0) // self.gpus_per_slot)
            slots = int(slots)
            if hostname and slots > 0:
                mapping[hostname] = slots
        return mapping
