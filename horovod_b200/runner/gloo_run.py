"""Launches the ranks of a job with the TCP/HTTP rendezvous ("gloo"
controller in the reference's vocabulary): starts the rendezvous server,
computes every slot's environment, runs the command on each slot locally or
through ssh, and kills everything as soon as one rank fails.

Parity: horovod/runner/gloo_run.py:65-284.
"""
import os
import shlex
import signal
import socket
import sys
import threading

from horovod_b200.runner.common import hosts as hosts_mod
from horovod_b200.runner.common import safe_shell_exec
from horovod_b200.runner.http.http_server import RendezvousServer, local_ip_for
from horovod_b200.runner.util import threads

LOCAL_NAMES = {"localhost", "127.0.0.1", "::1"}


def is_local_host(hostname):
    if hostname in LOCAL_NAMES:
        return True
    try:
        return hostname in (socket.gethostname(), socket.getfqdn())
    except OSError:
        return False


def create_slot_env_vars(slot_info):
    return {
        "HOROVOD_HOSTNAME": slot_info.hostname,
        "HOROVOD_RANK": str(slot_info.rank),
        "HOROVOD_SIZE": str(slot_info.size),
        "HOROVOD_LOCAL_RANK": str(slot_info.local_rank),
        "HOROVOD_LOCAL_SIZE": str(slot_info.local_size),
        "HOROVOD_CROSS_RANK": str(slot_info.cross_rank),
        "HOROVOD_CROSS_SIZE": str(slot_info.cross_size),
    }


def create_run_env_vars(server_ip, port, nics=None, elastic=False):
    env = {
        "HOROVOD_GLOO_RENDEZVOUS_ADDR": server_ip,
        "HOROVOD_GLOO_RENDEZVOUS_PORT": str(port),
        "HOROVOD_CONTROLLER": "gloo",
        "HOROVOD_CPU_OPERATIONS": "gloo",
    }
    if nics:
        iface = list(nics)[0]
        env["HOROVOD_GLOO_IFACE"] = iface
        env["NCCL_SOCKET_IFNAME"] = ",".join(nics)
    if elastic:
        env["HOROVOD_ELASTIC"] = "1"
    return env


def get_ssh_command(local_command, host, port=None, identity_file=None):
    opts = "-o PasswordAuthentication=no -o StrictHostKeyChecking=no"
    if port:
        opts += " -p %d" % port
    if identity_file:
        opts += " -i %s" % identity_file
    return "ssh %s %s %s" % (opts, host, shlex.quote(local_command))


_EXPORT_SKIP = {"BASH_FUNC", "OLDPWD", "_", "SHLVL", "PWD"}


def slot_command(command, slot_env, run_env, base_env, slot_info, settings):
    """Shell line that runs ``command`` for one slot (with ssh for remote
    hosts, where the whole environment has to travel on the command line)."""
    cmd = " ".join(shlex.quote(c) for c in command) if not isinstance(command, str) else command
    if is_local_host(slot_info.hostname):
        return cmd
    exports = []
    for k, v in {**base_env, **run_env, **slot_env}.items():
        if any(k.startswith(s) for s in _EXPORT_SKIP) or not k.replace("_", "").isalnum():
            continue
        exports.append("%s=%s" % (k, shlex.quote(v)))
    remote = "cd %s > /dev/null 2>&1 ; env %s %s" % (shlex.quote(os.getcwd()),
                                                       " ".join(exports), cmd)
    return get_ssh_command(remote, slot_info.hostname, getattr(settings, "ssh_port", None),
                           getattr(settings, "ssh_identity_file", None))


def _exec_slot(command, slot_info, run_env, base_env, settings, events):
    slot_env = create_slot_env_vars(slot_info)
    env = dict(base_env)
    env.update(run_env)
    env.update(slot_env)
    line = slot_command(command, slot_env, run_env, base_env, slot_info, settings)
    out, err, opened = sys.stdout, sys.stderr, []
    if getattr(settings, "output_filename", None):
        d = os.path.join(settings.output_filename, "rank.%0*d" % (len(str(slot_info.size)),
                                                                   slot_info.rank))
        os.makedirs(d, exist_ok=True)
        out = open(os.path.join(d, "stdout"), "w")
        err = open(os.path.join(d, "stderr"), "w")
        opened = [out, err]
    try:
        code = safe_shell_exec.execute(
            line, env=env, stdout=out, stderr=err, index=slot_info.rank, events=events,
            prefix_output_with_timestamp=getattr(settings, "prefix_output_with_timestamp",
                                                 False))
    finally:
        for f in opened:
            f.close()
    return code


def launch_gloo(command, exec_command, settings, nics, env, server_ip):
    """Static job: returns when every rank has exited; raises RuntimeError
    naming the first failed rank otherwise."""
    host_alloc_plan = hosts_mod.get_host_assignments(hosts_mod.parse_hosts(settings.hosts),
                                                     settings.num_proc)
    server = RendezvousServer(settings.verbose)
    port = server.start()
    server.init(host_alloc_plan)
    run_env = create_run_env_vars(server_ip, port, nics)

    failure = threading.Event()
    old = {}

    def on_signal(signum, frame):
        failure.set()
    if threading.current_thread() is threading.main_thread():
        for s in (signal.SIGINT, signal.SIGTERM):
            old[s] = signal.signal(s, on_signal)

    def run_slot(slot_info):
        code = exec_command(command, slot_info, run_env, env, settings, [failure])
        if code != 0:
            failure.set()  # first failure takes the job down
        return code, slot_info

    try:
        results = threads.execute_function_multithreaded(
            run_slot, [(s,) for s in host_alloc_plan], block_until_all_done=True)
    finally:
        for s, h in old.items():
            signal.signal(s, h)
        server.stop()
    failed = [(code, s) for code, s in results.values() if code != 0]
    if failed:
        # Report the rank that failed on its own, not the ones killed after it.
        failed.sort(key=lambda cs: (cs[0] in (143, 137, -15, -9, 128 + 15, 128 + 9), cs[1].rank))
        code, slot = failed[0]
        raise RuntimeError("Horovod detected that one or more processes exited with non-zero "
                           "status, thus causing the job to be terminated. The first process "
                           "to do so was:\nProcess name: %d\nExit code: %d\n"
                           % (slot.rank, code))


def gloo_run(settings, nics, env, server_ip, command):
    launch_gloo(command, _exec_slot, settings, nics, env, server_ip)


def launch_gloo_elastic(command, exec_command, settings, env, get_common_interfaces,
                        rendezvous=None):
    """Elastic job: an ElasticDriver keeps the set of workers in line with
    host discovery and re-runs rendezvous on every change."""
    from horovod_b200.runner.elastic.driver import ElasticDriver
    from horovod_b200.runner.elastic.rendezvous import attach_elastic_rendezvous

    server = rendezvous or RendezvousServer(settings.verbose)
    driver = ElasticDriver(server, settings.discovery, settings.min_np, settings.max_np,
                           timeout=settings.elastic_timeout, reset_limit=settings.reset_limit,
                           verbose=settings.verbose)
    port = server.start()
    attach_elastic_rendezvous(server, driver)
    nics = get_common_interfaces(driver) if get_common_interfaces else None
    server_ip = local_ip_for() if not all(
        is_local_host(h) for h in driver.host_manager.current_hosts.host_slots) else "127.0.0.1"
    run_env = create_run_env_vars(server_ip, port, nics, elastic=True)

    def run_slot(slot_info, events):
        # A new worker joins the rendezvous round during which it is started.
        env_now = dict(run_env, HOROVOD_ELASTIC_ROUND=str(driver.rendezvous_round()))
        return exec_command(command, slot_info, env_now, env, settings, events)

    try:
        driver.start(settings.num_proc, run_slot)
        res = driver.get_results()
        driver.stop()
    finally:
        server.stop()
    if res.error_message is not None:
        raise RuntimeError(res.error_message)
    for name, value in sorted(res.worker_results.items(), key=lambda item: item[1][1]):
        exit_code, _ts = value
        if exit_code != 0:
            raise RuntimeError("Horovod detected that one or more processes exited with "
                               "non-zero status, thus causing the job to be terminated. The "
                               "first process to do so was:\nProcess name: %s\nExit code: %d\n"
                               % (name, exit_code))


def gloo_run_elastic(settings, env, command):
    launch_gloo_elastic(command, _exec_slot, settings, env, None)
