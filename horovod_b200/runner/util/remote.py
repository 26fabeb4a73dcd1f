"""The command line that runs a command on another host.
Parity: horovod/runner/util/remote.py."""
from horovod_b200.runner.common import env as env_util

SSH_COMMAND_PREFIX = "ssh -o PasswordAuthentication=no -o StrictHostKeyChecking=no"


def get_ssh_command(local_command, host, port=None, identity_file=None, timeout_s=None):
    parts = [SSH_COMMAND_PREFIX, host]
    if port is not None:
        parts.append("-p %s" % port)
    if identity_file is not None:
        parts.append("-i %s" % identity_file)
    if timeout_s is not None:
        parts.append("-o ConnectTimeout=%s" % timeout_s)
    parts.append(local_command)
    return " ".join(parts)


def get_remote_command(local_command, host, port=None, identity_file=None, timeout_s=None):
    """ssh, or Kubeflow's exec wrapper when the MPI operator configured it."""
    if env_util.is_kubeflow_mpi():
        return "%s %s %s" % (env_util.KUBEFLOW_MPI_EXEC, host, local_command)
    return get_ssh_command(local_command, host, port, identity_file, timeout_s)
