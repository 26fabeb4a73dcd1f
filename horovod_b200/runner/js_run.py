"""Launch through IBM LSF ``jsrun``: builds the resource-set rankfile and the
jsrun command line.

Parity: horovod/runner/js_run.py:32-146, util/lsf.py:26-103.
"""
import os
import shlex
import sys
import tempfile

from horovod_b200.runner.common import hosts as hosts_mod
from horovod_b200.runner.common import safe_shell_exec


class LSFUtils:
    """What the LSF environment says about the allocation."""

    @staticmethod
    def using_lsf():
        return "LSB_JOBID" in os.environ

    @staticmethod
    def get_compute_hosts():
        hosts = os.environ.get("LSB_MCPU_HOSTS", "").split()
        pairs = list(zip(hosts[0::2], hosts[1::2]))
        # the first entry is the launch node
        return [h for h, _ in pairs[1:]] if len(pairs) > 1 else [h for h, _ in pairs]

    @staticmethod
    def get_num_gpus():
        return int(os.environ.get("HOROVOD_LSF_GPUS_PER_HOST", "4"))

    @staticmethod
    def get_num_cores():
        return int(os.environ.get("HOROVOD_LSF_CORES_PER_HOST", "40"))

    @staticmethod
    def get_num_threads():
        return int(os.environ.get("HOROVOD_LSF_THREADS_PER_CORE", "4"))


def is_jsrun_installed():
    """Whether the LSF launcher ``jsrun`` is on PATH."""
    import shutil
    return shutil.which("jsrun") is not None


def generate_jsrun_rankfile(settings, path=None):
    """One resource set (one GPU and its share of cores) per rank."""
    cores = LSFUtils.get_num_cores() // max(1, LSFUtils.get_num_gpus())
    threads = LSFUtils.get_num_threads()
    if path is None:
        fd, path = tempfile.mkstemp(prefix="hvd_jsrun_", suffix=".rf")
        os.close(fd)
    remaining = settings.num_proc
    with open(path, "w") as f:
        f.write("overlapping_rs: allow\ncpu_index_using: logical\n")
        rank = 0
        for host in hosts_mod.parse_hosts(settings.hosts):
            slots = min(host.slots, remaining)
            if slots <= 0:
                break
            f.write("\n")
            for s in range(slots):
                lo = s * cores * threads
                hi = lo + cores * threads - 1
                f.write("rank: %d: { hostname: %s; cpu: {%d-%d} ; gpu: * ; mem: * }\n"
                        % (rank, host.hostname, lo, hi))
                rank += 1
            remaining -= slots
    return path


def build_jsrun_command(settings, rankfile, env, command, addr, port):
    worker = "%s -m horovod_b200.runner.mpi_worker %s %d %s" % (
        shlex.quote(sys.executable), addr, port, " ".join(shlex.quote(c) for c in command))
    smpi = "--smpiargs '%s'" % (settings.extra_mpi_args or "-disable_gpu_hooks")
    out = ""
    if settings.output_filename:
        out = "--stdio_stderr %s --stdio_stdout %s" % (settings.output_filename,
                                                       settings.output_filename)
    binding = settings.binding_args or ""
    return " ".join(p for p in ["jsrun", "--erf_input %s" % rankfile, out, smpi, binding,
                                worker] if p)


def js_run(settings, nics, env, command, stdout=None, stderr=None):
    import shutil
    if shutil.which("jsrun") is None:
        raise Exception("horovodrun could not find jsrun; --jsrun needs an LSF allocation.")
    from horovod_b200.runner.http.http_server import RendezvousServer, local_ip_for
    server = RendezvousServer()
    port = server.start()
    server.init(hosts_mod.get_host_assignments(hosts_mod.parse_hosts(settings.hosts),
                                               settings.num_proc))
    try:
        rankfile = generate_jsrun_rankfile(settings)
        line = build_jsrun_command(settings, rankfile, env, command, local_ip_for(), port)
        code = safe_shell_exec.execute(line, env=env, stdout=stdout, stderr=stderr)
    finally:
        server.stop()
    if code != 0:
        raise RuntimeError("jsrun failed with exit code %d" % code)
