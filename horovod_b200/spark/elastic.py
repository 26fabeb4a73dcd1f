"""``horovod_b200.spark.run_elastic(fn, ...)``: an elastic job whose workers
are Spark tasks. ``max_np`` tasks are started as one (non-barrier) stage; each
registers with a coordinator on the driver and then asks it for work. The
elastic driver (the same one ``horovodrun`` uses) sees the registered tasks as
hosts and slots; when it wants a worker in a slot it hands that slot's
environment to a free task on that host, the task runs ``fn`` and reports its
result. Tasks that die simply stop asking; Spark restarts them and they
register again, which the driver notices as a host change.

Communication is pull-based (tasks call the driver, never the other way
round), over the launcher's HMAC-signed RPC
(``horovod_b200/runner/common/network.py``), so executors need no listening
ports. ``pyspark`` is imported at call time.

Parity: horovod/spark/runner.py:308-429 (run_elastic),
horovod/spark/driver/host_discovery.py (SparkDriverHostDiscovery).
"""
import os
import socket
import threading
import time

from horovod_b200.runner.common import network, secret
from horovod_b200.runner.elastic.discovery import HostDiscovery


class _Register:
    def __init__(self, index, host):
        self.index, self.host = index, host


class _NextAssignment:
    def __init__(self, index):
        self.index = index


class _Report:
    def __init__(self, index, exit_code, result):
        self.index, self.exit_code, self.result = index, exit_code, result


class _Assignment:
    """env: the worker's environment; None = nothing yet, ask again;
    finished: the job is over, the task may end."""

    def __init__(self, env=None, finished=False):
        self.env, self.finished = env, finished


class TaskCoordinator(network.BasicService, HostDiscovery):
    """Driver side: registry of live tasks (which doubles as host discovery)
    and the hand-over of slots to tasks."""

    NAME = "spark elastic coordinator"
    STALE_SECONDS = 10.0  # a task that has not asked for this long counts as gone

    def __init__(self, key, nics=None):
        self._lock = threading.Condition()
        self._tasks = {}      # index -> {"host", "seen", "busy", "env", "report"}
        self._finished = False
        network.BasicService.__init__(self, self.NAME, key, nics)

    # ---- RPC -----------------------------------------------------------------
    def _handle(self, req, client_address):
        if isinstance(req, _Register):
            with self._lock:
                self._tasks[req.index] = {"host": req.host, "seen": time.time(), "busy": False,
                                          "env": None, "report": None}
                self._lock.notify_all()
            return network.AckResponse()
        if isinstance(req, _NextAssignment):
            with self._lock:
                task = self._tasks.get(req.index)
                if self._finished or task is None:
                    return _Assignment(finished=self._finished)
                task["seen"] = time.time()
                env, task["env"] = task["env"], None
                return _Assignment(env=env)
        if isinstance(req, _Report):
            with self._lock:
                task = self._tasks.get(req.index)
                if task is not None:
                    task["report"] = (req.exit_code, req.result)
                    task["seen"] = time.time()
                    self._lock.notify_all()
            return network.AckResponse()
        return network.BasicService._handle(self, req, client_address)

    # ---- host discovery (what the elastic driver polls) ----------------------
    def find_available_hosts_and_slots(self):
        now = time.time()
        hosts = {}
        with self._lock:
            for task in self._tasks.values():
                if task["busy"] or now - task["seen"] <= self.STALE_SECONDS:
                    hosts[task["host"]] = hosts.get(task["host"], 0) + 1
        return hosts

    # ---- what the elastic driver's worker function uses ----------------------
    def run_in_slot(self, slot_info, env, events, poll=0.2):
        """Gives ``env`` to a free task on the slot's host and waits for its
        report. Returns (exit code, result); exit code 1 when no task took
        the slot or the job is being stopped."""
        with self._lock:
            free = [i for i, t in sorted(self._tasks.items())
                    if t["host"] == slot_info.hostname and not t["busy"]]
            if not free:
                return 1, None
            index = free[0]
            task = self._tasks[index]
            task.update(busy=True, env=env, report=None)
        try:
            while True:
                with self._lock:
                    if task["report"] is not None:
                        return task["report"]
                    self._lock.wait(poll)
                if any(e.is_set() for e in events or []):
                    return 1, None
        finally:
            with self._lock:
                task["busy"] = False
                task["env"] = None

    def wait_for_tasks(self, count, timeout):
        deadline = time.time() + timeout
        with self._lock:
            while len(self._tasks) < count:
                left = deadline - time.time()
                if left <= 0:
                    raise TimeoutError("Only %d of %d Spark tasks registered within %d s."
                                       % (len(self._tasks), count, timeout))
                self._lock.wait(left)

    def finish(self):
        with self._lock:
            self._finished = True
            self._lock.notify_all()


class _CoordinatorClient(network.BasicClient):
    def __init__(self, addresses, key):
        super().__init__(TaskCoordinator.NAME, addresses, key)

    def register(self, index, host):
        self._send(_Register(index, host))

    def next_assignment(self, index):
        return self._send(_NextAssignment(index))

    def report(self, index, exit_code, result):
        self._send(_Report(index, exit_code, result))


def _task_loop(index, addresses, key, fn, args, kwargs, poll=0.2):
    """Body of one Spark task: register, then run whatever slots the driver
    hands over until the job is finished."""
    client = _CoordinatorClient(addresses, key)
    client.register(index, socket.gethostname())
    while True:
        assignment = client.next_assignment(index)
        if assignment.finished:
            return
        if assignment.env is None:
            time.sleep(poll)
            continue
        os.environ.update(assignment.env)
        try:
            result, code = fn(*args, **kwargs), 0
        except SystemExit as e:
            # the function ended its "process" (an elastic worker that was removed
            # exits with 0): the Spark task itself lives on for later assignments
            result, code = None, (e.code if isinstance(e.code, int) else 0 if e.code is None else 1)
        except Exception as e:  # noqa: BLE001 - the driver decides what a failure means
            result, code = repr(e), 1
        client.report(index, code, result)


def run_elastic(fn, args=(), kwargs=None, num_proc=None, min_np=None, max_np=None,
                start_timeout=None, elastic_timeout=600, reset_limit=None, env=None, nics=None,
                verbose=1):
    """Runs ``fn(*args, **kwargs)`` (which uses ``hvd.elastic.run`` inside) on
    between ``min_np`` and ``max_np`` Spark tasks and returns the results of
    the last round's workers ordered by rank."""
    from horovod_b200.spark.runner import _require_pyspark
    from horovod_b200.runner.elastic.driver import ElasticDriver
    from horovod_b200.runner.elastic.rendezvous import attach_elastic_rendezvous
    from horovod_b200.runner.gloo_run import create_run_env_vars, create_slot_env_vars
    from horovod_b200.runner.http.http_server import RendezvousServer, local_ip_for
    pyspark = _require_pyspark()
    kwargs = kwargs or {}
    if start_timeout is None:
        # how long to wait for min_np tasks to register (horovod/spark/runner.py:219-223)
        start_timeout = int(os.environ.get("HOROVOD_SPARK_START_TIMEOUT", "600"))
    spark_context = pyspark.SparkContext._active_spark_context
    if spark_context is None:
        raise Exception("Could not find an active SparkContext, are you running in a "
                        "PySpark session?")
    num_proc = num_proc or spark_context.defaultParallelism
    min_np = min_np or num_proc
    max_np = max_np or num_proc
    if not min_np <= num_proc <= max_np:
        raise ValueError("need min_np <= num_proc <= max_np, got %d, %d, %d"
                         % (min_np, num_proc, max_np))

    key = secret.make_secret_key()
    coordinator = TaskCoordinator(key, nics)
    addresses = coordinator.addresses()
    rendezvous = RendezvousServer(verbose)
    driver = ElasticDriver(rendezvous, coordinator, min_np, max_np, timeout=elastic_timeout,
                           reset_limit=reset_limit, verbose=verbose)
    port = rendezvous.start()
    attach_elastic_rendezvous(rendezvous, driver)
    run_env = create_run_env_vars(local_ip_for(), port, nics, elastic=True)
    run_env.update({k: str(v) for k, v in (env or {}).items()})
    results = {}

    def spark_stage():
        def task(index, _iterator):
            from horovod_b200.spark import task as task_info
            try:
                from pyspark import TaskContext
                task_info.set_resources(task_info.resources_of(TaskContext.get()))
            except ImportError:  # a pyspark without TaskContext: no resource information
                task_info.set_resources({})
            _task_loop(index, addresses, key, fn, args, kwargs)
            yield index
        spark_context.range(0, numSlices=max_np).mapPartitionsWithIndex(task).collect()

    stage = threading.Thread(target=spark_stage, daemon=True, name="hvd-spark-elastic-stage")
    stage.start()

    def run_slot(slot_info, events):
        slot_env = dict(run_env)
        slot_env.update(create_slot_env_vars(slot_info))
        slot_env["HOROVOD_ELASTIC_ROUND"] = str(driver.rendezvous_round())
        code, value = coordinator.run_in_slot(slot_info, slot_env, events)
        if code == 0:
            results[slot_info.rank] = value
        return code

    try:
        coordinator.wait_for_tasks(min_np, start_timeout)
        driver.start(num_proc, run_slot)
        outcome = driver.get_results()
        driver.stop()
    finally:
        coordinator.finish()
        stage.join(timeout=30)
        rendezvous.stop()
        coordinator.shutdown()
    if outcome.error_message is not None:
        raise RuntimeError(outcome.error_message)
    failed = sorted((ts, name, code) for name, (code, ts) in outcome.worker_results.items()
                    if code != 0)
    if failed:
        raise RuntimeError("Elastic Spark job ended with failed workers; the first was %s "
                           "(exit code %d)." % (failed[0][1], failed[0][2]))
    return [results[r] for r in sorted(results)]
