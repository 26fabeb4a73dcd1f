"""What the launcher needs to know about the environment: which variables are
forwarded to remote ranks, and the rank/size a process was started with by
whichever launcher (this one, Open MPI, PMI).
Parity: horovod/runner/common/util/env.py."""
import os
import re

from horovod_b200.runner.common import secret

LOG_LEVEL_STR = ["FATAL", "ERROR", "WARNING", "INFO", "DEBUG", "TRACE"]
KUBEFLOW_MPI_EXEC = "/etc/mpi/kubexec.sh"
# Names that are never forwarded to other hosts: exported shell functions,
# the previous working directory and the job's secret.
IGNORE_REGEXES = {"BASH_FUNC_.*", "OLDPWD", secret.HOROVOD_SECRET_KEY}
_IGNORED = [re.compile(pattern) for pattern in sorted(IGNORE_REGEXES)]
# (rank variable, size variable) of the launchers a rank may come from.
_LAUNCHER_VARS = (("HOROVOD_RANK", "HOROVOD_SIZE"),
                  ("OMPI_COMM_WORLD_RANK", "OMPI_COMM_WORLD_SIZE"),
                  ("PMI_RANK", "PMI_SIZE"))


def is_exportable(name):
    """False for variables that must stay on this host."""
    for pattern in _IGNORED:
        if pattern.match(name):
            return False
    return True


def get_env_rank_and_size():
    """(rank, size) from the first launcher that set both of its variables;
    (0, 1) for a process that no launcher started. One variable of a pair
    without the other is an error."""
    for pair in _LAUNCHER_VARS:
        found = [os.environ.get(name) for name in pair]
        if all(v is not None for v in found):
            return int(found[0]), int(found[1])
        if any(v is not None for v in found):
            raise RuntimeError("Could not determine process rank and size: only one of %s and "
                               "%s found in environment" % pair)
    return 0, 1


def is_kubeflow_mpi():
    """Whether Open MPI was told to reach other hosts through Kubeflow's wrapper."""
    return os.environ.get("OMPI_MCA_plm_rsh_agent", "") == KUBEFLOW_MPI_EXEC
