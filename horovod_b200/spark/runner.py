"""``horovod_b200.spark.run(fn, ...)``: runs ``fn`` on ``num_proc`` Spark tasks
of one barrier stage as the ranks of one job and returns the results by
rank. The tasks learn each other's hosts through the barrier context, derive
their local/cross coordinates from them and meet at a rendezvous server on
the driver. ``pyspark`` (3.0 or newer, for BarrierTaskContext.allGather) is
imported at call time; the tests drive run() through a stand-in pyspark
module, since pyspark itself is not installed here.
Parity: horovod/spark/runner.py:197-305 (run). The elastic variant is in
horovod_b200/spark/elastic.py, the estimator for PyTorch models in
horovod_b200/spark/torch.
"""
import os
import socket


def _require_pyspark():
    try:
        import pyspark
        return pyspark
    except ImportError as e:  # pragma: no cover - depends on the environment
        raise ImportError("horovod_b200.spark needs the `pyspark` package, which is not "
                          "installed in this environment.") from e


def _coordinates(hostnames, rank):
    """(local_rank, local_size, cross_rank, cross_size) of ``rank`` given the
    host of every rank: ranks on one host are numbered in rank order; the
    cross rank counts the hosts (in order of first appearance) that have that
    local rank."""
    by_host = {}
    for r, h in enumerate(hostnames):
        by_host.setdefault(h, []).append(r)
    mine = by_host[hostnames[rank]]
    local_rank = mine.index(rank)
    hosts_with = [h for h, ranks in by_host.items() if len(ranks) > local_rank]
    return local_rank, len(mine), hosts_with.index(hostnames[rank]), len(hosts_with)


def run(fn, args=(), kwargs=None, num_proc=None, start_timeout=None, use_mpi=None, use_gloo=None,
        env=None, extra_env=None, nics=None, verbose=1):
    """Runs ``fn(*args, **kwargs)`` on ``num_proc`` ranks inside Spark tasks;
    returns the list of results ordered by rank. If the tasks have not all
    started within ``start_timeout`` seconds (default: the environment
    variable HOROVOD_SPARK_START_TIMEOUT, else 600) the Spark job is cancelled
    and an exception says that the cluster lacks the resources for
    ``num_proc`` simultaneous tasks. ``env`` (or ``extra_env``) is added to
    every rank's environment; ``nics`` names the network interfaces the ranks
    may use; the ranks always meet through this package's TCP rendezvous, so
    ``use_mpi=True`` is refused."""
    import threading
    if use_mpi:
        raise ValueError("horovod_b200.spark.run has no MPI controller; leave use_mpi unset "
                         "(the ranks rendezvous over TCP, as with use_gloo=True).")
    pyspark = _require_pyspark()
    from pyspark import BarrierTaskContext
    from horovod_b200.runner.http.http_client import put_data_into_kvstore
    from horovod_b200.runner.http.http_server import RendezvousServer, local_ip_for
    kwargs = kwargs or {}
    if start_timeout is None:
        start_timeout = int(os.environ.get("HOROVOD_SPARK_START_TIMEOUT", "600"))
    spark_context = pyspark.SparkContext._active_spark_context
    if spark_context is None:
        raise Exception("Could not find an active SparkContext, are you running in a "
                        "PySpark session?")
    if num_proc is None:
        num_proc = spark_context.defaultParallelism
        if verbose >= 1:
            print("Running %d processes (inferred from spark.default.parallelism)..." % num_proc)
    server = RendezvousServer(verbose)
    port = server.start()
    server.init([None] * num_proc)
    driver_ip = local_ip_for()
    extra = dict(env or {})
    extra.update(extra_env or {})
    if nics:
        names = ",".join(sorted(nics)) if not isinstance(nics, str) else nics
        extra.setdefault("HOROVOD_GLOO_IFACE", names.split(",")[0])
        extra.setdefault("NCCL_SOCKET_IFNAME", names)

    def task(index, _iterator):
        ctx = BarrierTaskContext.get()
        hostnames = ctx.allGather(socket.gethostname())
        rank = ctx.partitionId()
        # the barrier has let every task through: tell the driver that the job has started
        put_data_into_kvstore(driver_ip, port, _STARTED_SCOPE, str(rank), b"1")
        from horovod_b200.spark import task as task_info
        task_info.set_resources(task_info.resources_of(ctx))
        local_rank, local_size, cross_rank, cross_size = _coordinates(hostnames, rank)
        os.environ.update({k: str(v) for k, v in extra.items()})
        os.environ.update({
            "HOROVOD_RANK": str(rank), "HOROVOD_SIZE": str(len(hostnames)),
            "HOROVOD_LOCAL_RANK": str(local_rank), "HOROVOD_LOCAL_SIZE": str(local_size),
            "HOROVOD_CROSS_RANK": str(cross_rank), "HOROVOD_CROSS_SIZE": str(cross_size),
            "HOROVOD_HOSTNAME": hostnames[rank],
            "HOROVOD_GLOO_RENDEZVOUS_ADDR": driver_ip,
            "HOROVOD_GLOO_RENDEZVOUS_PORT": str(port),
            "HOROVOD_CONTROLLER": "gloo", "HOROVOD_CPU_OPERATIONS": "gloo",
        })
        yield rank, fn(*args, **kwargs)

    group = "horovod_b200.spark.run.%d" % port
    outcome = {}

    def stage():
        try:
            if hasattr(spark_context, "setJobGroup"):
                spark_context.setJobGroup(group, "horovod_b200.spark.run", interruptOnCancel=True)
            outcome["pairs"] = spark_context.range(0, numSlices=num_proc).barrier() \
                .mapPartitionsWithIndex(task).collect()
        except BaseException as e:  # noqa: BLE001 - re-raised in the caller's thread
            outcome["error"] = e

    worker = threading.Thread(target=stage, daemon=True, name="hvd-spark-stage")
    try:
        worker.start()
        if not _wait_for_start(server, worker, start_timeout):
            if hasattr(spark_context, "cancelJobGroup"):
                spark_context.cancelJobGroup(group)
            raise Exception(
                "Timed out waiting for the Spark tasks to start. Please check that you have "
                "enough resources to run all %d processes at the same time: each process runs "
                "in its own Spark task. Raise start_timeout (now %d s) if the cluster is only "
                "slow to hand out executors." % (num_proc, start_timeout))
        worker.join()
    finally:
        server.stop()
    if "error" in outcome:
        raise outcome["error"]
    return [result for _rank, result in sorted(outcome["pairs"], key=lambda p: p[0])]


_STARTED_SCOPE = "spark_task_started"


def _wait_for_start(server, worker, timeout, poll=0.05):
    """True once a task has checked in (the barrier releases all of them
    together) or the stage has ended; False when ``timeout`` seconds passed
    first."""
    import time
    deadline = time.monotonic() + timeout
    while time.monotonic() < deadline:
        if not worker.is_alive() or server.get(_STARTED_SCOPE, "0") is not None:
            return True
        time.sleep(poll)
    return not worker.is_alive() or server.get(_STARTED_SCOPE, "0") is not None
