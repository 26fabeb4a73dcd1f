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


class ElasticRayExecutor:
    """Elastic job on a Ray cluster: the elastic driver keeps as many workers
    alive as the cluster's nodes have slots (between ``min_np`` and
    ``max_np``), starting each worker as a Ray task pinned to its node, and
    re-runs the rendezvous whenever nodes come or go.

        settings = ElasticRayExecutor.create_settings(min_np=2, max_np=8)
        executor = ElasticRayExecutor(settings, use_gpu=True, cpus_per_slot=2)
        executor.start()
        results = executor.run(train_fn)   # train_fn uses hvd.elastic.run inside

    ``run`` returns the values ``train_fn`` returned on the workers of the last
    round, ordered by rank. Parity: horovod/ray/elastic.py:96-465.
    """

    @staticmethod
    def create_settings(min_np=1, max_np=None, reset_limit=None, elastic_timeout=600,
                        timeout_s=30, ssh_identity_file=None, nics=None, verbose=1, **kwargs):
        from horovod_b200.runner.common.settings import ElasticSettings
        from horovod_b200.runner.common.timeout import Timeout
        return ElasticSettings(discovery=None, min_np=min_np, max_np=max_np,
                               elastic_timeout=elastic_timeout, reset_limit=reset_limit,
                               num_proc=min_np, verbose=verbose,
                               ssh_identity_file=ssh_identity_file, nics=nics,
                               start_timeout=Timeout(timeout_s,
                                                     "Timed out waiting for {activity}."),
                               **kwargs)

    def __init__(self, settings, use_gpu=False, cpus_per_slot=1, gpus_per_slot=None,
                 env_vars=None, override_discovery=True):
        if gpus_per_slot and not use_gpu:
            raise ValueError("gpus_per_slot is set, but use_gpu is False.")
        if use_gpu and gpus_per_slot is not None and gpus_per_slot < 1:
            raise ValueError("gpus_per_slot must be at least 1 with use_gpu.")
        self.settings = settings
        self.use_gpu = use_gpu
        self.cpus_per_slot = cpus_per_slot
        self.gpus_per_slot = gpus_per_slot or (1 if use_gpu else 0)
        self.env_vars = dict(env_vars or {})
        if override_discovery or getattr(settings, "discovery", None) is None:
            settings.discovery = RayHostDiscovery(use_gpu=use_gpu, cpus_per_slot=cpus_per_slot,
                                                  gpus_per_slot=self.gpus_per_slot or 1)
        self.driver = None
        self.rendezvous = None
        self._run_env = None
        self._results = {}

    def start(self, advertise_ip=None):
        """Starts the rendezvous server and the elastic driver."""
        from horovod_b200.runner.elastic.driver import ElasticDriver
        from horovod_b200.runner.elastic.rendezvous import attach_elastic_rendezvous
        from horovod_b200.runner.gloo_run import create_run_env_vars
        from horovod_b200.runner.http.http_server import RendezvousServer, local_ip_for
        s = self.settings
        self.rendezvous = RendezvousServer(getattr(s, "verbose", 0) or 0)
        self.driver = ElasticDriver(self.rendezvous, s.discovery, s.min_np, s.max_np,
                                    timeout=getattr(s, "elastic_timeout", None),
                                    reset_limit=getattr(s, "reset_limit", None),
                                    verbose=getattr(s, "verbose", 0) or 0)
        port = self.rendezvous.start()
        attach_elastic_rendezvous(self.rendezvous, self.driver)
        self._run_env = create_run_env_vars(advertise_ip or local_ip_for(), port,
                                            getattr(s, "nics", None), elastic=True)

    def _slot_task(self, ray, worker_fn):
        """The function the driver calls for every slot it wants a worker in:
        runs ``worker_fn`` as a Ray task on the slot's node with the slot's
        environment and records what it returned."""
        from horovod_b200.runner.gloo_run import create_slot_env_vars

        def remote_body(env, fn):
            import os
            os.environ.update(env)
            try:
                return fn()
            except SystemExit as e:
                # an elastic worker that was removed from the job ends with exit
                # code 0; the Ray worker process must not go down with it
                if e.code in (0, None):
                    return None
                raise RuntimeError("the worker function exited with code %r" % (e.code,))

        def run_slot(slot_info, events):
            env = dict(self._run_env)
            env.update(create_slot_env_vars(slot_info))
            env["HOROVOD_ELASTIC_ROUND"] = str(self.driver.rendezvous_round())
            env.update({k: str(v) for k, v in self.env_vars.items()})
            task = ray.remote(remote_body).options(
                num_cpus=self.cpus_per_slot, num_gpus=self.gpus_per_slot,
                resources={"node:%s" % slot_info.hostname: 0.01})
            ref = task.remote(env, worker_fn)
            # Poll, so that the end of the job (events) stops the wait.
            while True:
                done, _ = ray.wait([ref], timeout=0.5)
                if done:
                    break
                if any(e.is_set() for e in events or []):
                    ray.cancel(ref, force=True)
                    return 1
            try:
                value = ray.get(ref)
            except Exception:  # the worker failed or its node went away
                return 1
            self._results[slot_info.rank] = value
            return 0

        return run_slot

    def run(self, worker_fn):
        """Runs ``worker_fn`` on every slot until the job ends; returns the
        workers' return values ordered by rank."""
        from horovod_b200.ray.runner import _require_ray
        ray = _require_ray()
        if self.driver is None:
            self.start()
        self._results = {}
        try:
            self.driver.start(self.settings.num_proc, self._slot_task(ray, worker_fn))
            outcome = self.driver.get_results()
            self.driver.stop()
        finally:
            self.rendezvous.stop()
            self.driver = None
        if outcome.error_message is not None:
            raise RuntimeError(outcome.error_message)
        failed = sorted((ts, name, code) for name, (code, ts) in outcome.worker_results.items()
                        if code != 0)
        if failed:
            raise RuntimeError("Elastic Ray job ended with failed workers; the first was %s "
                               "(exit code %d)." % (failed[0][1], failed[0][2]))
        return [self._results[r] for r in sorted(self._results)]
