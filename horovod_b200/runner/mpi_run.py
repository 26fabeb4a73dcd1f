"""Builds and runs an ``mpirun`` command line for jobs launched through MPI
(Open MPI, Spectrum MPI, MPICH, Intel MPI). The ranks still talk to each
other over this framework's TCP mesh; mpirun is only the process starter, and
its rank variables are translated by ``horovod_b200.runner.mpi_worker``.

Parity: horovod/runner/mpi_run.py:120-254.
"""
import os
import shlex
import subprocess
import sys

from horovod_b200.runner.common import hosts as hosts_mod
from horovod_b200.runner.common import safe_shell_exec

_OMPI_IMPL, _SMPI_IMPL, _MPICH_IMPL, _IMPI_IMPL = "OpenMPI", "SpectrumMPI", "MPICH", "IntelMPI"
_UNKNOWN_IMPL, _MISSING_IMPL = "Unknown", "Missing"

_OMPI_FLAGS = ["-mca pml ob1", "-mca btl ^openib"]
_SMPI_FLAGS = []
_SMPI_FLAGS_TCP = ["-tcp"]
_MPICH_FLAGS = []
_IMPI_FLAGS = []
_NO_BINDING_ARGS = ["-bind-to none", "-map-by slot"]
_SOCKET_BINDING_ARGS = ["-bind-to socket", "-map-by socket", "-rank-by core"]
_LARGE_CLUSTER_THRESHOLD = 64


def _exec(command):
    try:
        res = subprocess.run(command, stdout=subprocess.PIPE, stderr=subprocess.STDOUT,
                             text=True, timeout=30)
        return res.stdout, res.returncode
    except (OSError, subprocess.TimeoutExpired):
        return None, 127


def _get_mpi_implementation(env=None):
    """Which MPI the ``mpirun`` on PATH belongs to."""
    output, code = _exec(["mpirun", "--version"])
    if output is None:
        return _MISSING_IMPL
    if code != 0:
        return _UNKNOWN_IMPL
    if "Open MPI" in output or "OpenRTE" in output:
        return _OMPI_IMPL
    if "IBM Spectrum MPI" in output:
        return _SMPI_IMPL
    if "MPICH" in output or "HYDRA" in output:
        return _MPICH_IMPL
    if "Intel(R) MPI" in output:
        return _IMPI_IMPL
    return _UNKNOWN_IMPL


def _get_mpi_implementation_flags(tcp_flag, env=None):
    impl = _get_mpi_implementation(env)
    if impl == _OMPI_IMPL:
        return list(_OMPI_FLAGS), list(_NO_BINDING_ARGS), impl
    if impl == _SMPI_IMPL:
        flags = list(_SMPI_FLAGS_TCP) if tcp_flag else list(_SMPI_FLAGS)
        return flags, list(_SOCKET_BINDING_ARGS), impl
    if impl == _MPICH_IMPL:
        return list(_MPICH_FLAGS), [], impl
    if impl == _IMPI_IMPL:
        return list(_IMPI_FLAGS), [], impl
    return None, None, impl


def mpi_available(env=None):
    return _get_mpi_implementation(env) not in (_UNKNOWN_IMPL, _MISSING_IMPL)


def is_open_mpi(env=None):
    return _get_mpi_implementation(env) == _OMPI_IMPL


def is_spectrum_mpi(env=None):
    return _get_mpi_implementation(env) == _SMPI_IMPL


def is_mpich(env=None):
    return _get_mpi_implementation(env) == _MPICH_IMPL


def is_intel_mpi(env=None):
    return _get_mpi_implementation(env) == _IMPI_IMPL


def build_mpi_command(settings, nics, env, command, impl_flags, binding_args, impl,
                      rendezvous_addr, rendezvous_port):
    """Returns the full mpirun command line as a string."""
    hosts = settings.hosts
    host_names = [h.hostname for h in hosts_mod.parse_hosts(hosts)]
    flags = list(impl_flags)
    if impl == _OMPI_IMPL and len(host_names) >= _LARGE_CLUSTER_THRESHOLD:
        flags += ["-mca plm_rsh_no_tree_spawn true",
                  "-mca plm_rsh_num_concurrent %d" % len(host_names)]
    ssh_args = []
    if settings.ssh_port:
        ssh_args.append("-p %d" % settings.ssh_port)
    if settings.ssh_identity_file:
        ssh_args.append("-i %s" % settings.ssh_identity_file)
    if ssh_args and impl == _OMPI_IMPL:
        flags.append('-mca plm_rsh_args "%s"' % " ".join(ssh_args))
    if nics and impl == _OMPI_IMPL:
        flags.append("-mca btl_tcp_if_include %s" % ",".join(nics))
        flags.append("-x NCCL_SOCKET_IFNAME=%s" % ",".join(nics))
    binding = settings.binding_args if settings.binding_args else " ".join(binding_args)
    exported = sorted(k for k in env if k.startswith(("HOROVOD_", "NCCL_", "PYTHONPATH", "PATH",
                                                      "LD_LIBRARY_PATH", "CUDA_")))
    if impl in (_OMPI_IMPL, _SMPI_IMPL):
        env_args = " ".join("-x %s" % k for k in exported)
        host_arg = "-H %s" % hosts
        np_arg = "-np %d" % settings.num_proc
        extra = "--allow-run-as-root --tag-output"
    else:
        env_args = "-genvlist %s" % ",".join(exported) if exported else ""
        host_arg = "-hosts %s" % ",".join(host_names)
        np_arg = "-np %d" % settings.num_proc
        extra = "-prepend-rank" if impl == _MPICH_IMPL else "-l"
    worker = "%s -m horovod_b200.runner.mpi_worker %s %d %s" % (
        shlex.quote(sys.executable), rendezvous_addr, rendezvous_port,
        " ".join(shlex.quote(c) for c in command))
    parts = ["mpirun", extra, np_arg, host_arg, binding, " ".join(flags), env_args,
             settings.extra_mpi_args or "", worker]
    return " ".join(p for p in parts if p)


def mpi_run(settings, nics, env, command, stdout=None, stderr=None):
    impl_flags, binding_args, impl = _get_mpi_implementation_flags(settings.tcp_flag, env)
    if impl_flags is None:
        raise Exception("horovodrun could not find a usable mpirun (found: %s). Install "
                        "Open MPI 4.x, MPICH or Intel MPI, or launch without --mpi." % impl)
    from horovod_b200.runner.http.http_server import RendezvousServer, local_ip_for
    server = RendezvousServer()
    port = server.start()
    server.init(hosts_mod.get_host_assignments(hosts_mod.parse_hosts(settings.hosts),
                                               settings.num_proc))
    try:
        line = build_mpi_command(settings, nics, env, command, impl_flags, binding_args, impl,
                                 local_ip_for(), port)
        if settings.verbose >= 2:
            print(line)
        code = safe_shell_exec.execute(line, env=env, stdout=stdout, stderr=stderr)
    finally:
        server.stop()
    if code != 0:
        raise RuntimeError("mpirun failed with exit code %d" % code)
