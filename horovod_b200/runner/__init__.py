"""Programmatic launcher: ``horovod_b200.run(func, args=(), np=2)`` runs
``func`` on ``np`` ranks and returns the list of results ordered by rank.

The function is pickled into the launcher's key-value server; every worker
process (``python -m horovod_b200.runner.run_task``) fetches it, calls it and
stores its result under its rank.

Parity: horovod/runner/__init__.py:92-210, launch.py:594-614,
run_task.py:22, task_fn.py:23.
"""
import os
import sys

import cloudpickle


class _HorovodArgs:
    def __init__(self):
        self.np = 1
        self.check_build = None
        self.ssh_port = None
        self.ssh_identity_file = None
        self.disable_cache = None
        self.start_timeout = None
        self.nics = None
        self.output_filename = None
        self.verbose = None
        self.use_gloo = None
        self.use_mpi = None
        self.use_jsrun = None
        self.mpi_args = None
        self.tcp_flag = None
        self.binding_args = None
        self.hosts = None
        self.hostfile = None
        self.host_discovery_script = None
        self.min_np = None
        self.max_np = None
        self.slots = None
        self.elastic_timeout = None
        self.reset_limit = None
        self.config_file = None
        self.prefix_output_with_timestamp = False
        self.run_func = None
        self.command = None


def run(func, args=(), kwargs=None, np=1, min_np=None, max_np=None, slots=None,
        reset_limit=None, hosts=None, hostfile=None, start_timeout=None, ssh_port=None,
        ssh_identity_file=None, disable_cache=None, output_filename=None, verbose=None,
        use_gloo=None, use_mpi=None, mpi_args=None, network_interface=None,
        executable=None, env=None, elastic_timeout=None, host_discovery_script=None):
    """Runs ``func(*args, **kwargs)`` on ``np`` ranks; returns results by rank."""
    from horovod_b200.runner import launch
    from horovod_b200.runner.http.http_server import KVStoreServer

    kwargs = kwargs or {}
    hargs = _HorovodArgs()
    hargs.np = np
    hargs.min_np, hargs.max_np, hargs.slots = min_np, max_np, slots
    hargs.reset_limit, hargs.elastic_timeout = reset_limit, elastic_timeout
    hargs.hosts, hargs.hostfile = hosts, hostfile
    hargs.host_discovery_script = host_discovery_script
    hargs.start_timeout, hargs.ssh_port = start_timeout, ssh_port
    hargs.ssh_identity_file, hargs.disable_cache = ssh_identity_file, disable_cache
    hargs.output_filename, hargs.verbose = output_filename, verbose
    hargs.use_gloo, hargs.use_mpi, hargs.mpi_args = use_gloo, use_mpi, mpi_args
    hargs.nics = network_interface

    kv = KVStoreServer()
    port = kv.start_server()
    kv.put("runfunc", "func", cloudpickle.dumps((func, tuple(args), kwargs)))
    from horovod_b200.runner.gloo_run import is_local_host
    from horovod_b200.runner.common import hosts as hosts_mod
    host_list = [h.hostname for h in hosts_mod.parse_hosts(hosts)] if hosts else ["localhost"]
    if all(is_local_host(h) for h in host_list):
        addr = "127.0.0.1"
    else:
        from horovod_b200.runner.http.http_server import local_ip_for
        addr = local_ip_for(host_list[0])
    hargs.command = [executable or sys.executable, "-m", "horovod_b200.runner.run_task",
                     addr, str(port)]
    hargs.run_func = func
    old_env = None
    if env is not None:
        old_env = os.environ.copy()
        os.environ.update(env)
    try:
        launch._run(hargs)
        results = []
        size = None
        rank = 0
        while size is None or rank < size:
            blob = kv.get("runfunc_result", str(rank))
            if blob is None:
                if size is None:
                    raise RuntimeError("no results were returned by the workers")
                raise RuntimeError("rank %d returned no result" % rank)
            ok, payload, world = cloudpickle.loads(blob)
            size = world
            if not ok:
                raise RuntimeError("rank %d failed:\n%s" % (rank, payload))
            results.append(payload)
            rank += 1
        return results
    finally:
        kv.shutdown_server()
        if old_env is not None:
            os.environ.clear()
            os.environ.update(old_env)
