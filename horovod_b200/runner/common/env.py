"""What the launcher needs to know about the environment: which variables are
forwarded to remote ranks, and the rank/size a process was started with by
whichever launcher (this one, Open MPI, PMI).
Parity: horovod/runner/common/util/env.py."""
import os
import re

from horovod_b200.runner.common import secret

LOG_LEVEL_STR = ["FATAL", "ERROR", "WARNING", "INFO", "DEBUG", "TRACE"]

# Never forwarded: shell function exports, the previous directory, the job's secret.
IGNORE_REGEXES = {"BASH_FUNC_.*", "OLDPWD", secret.HOROVOD_SECRET_KEY}

KUBEFLOW_MPI_EXEC = "/etc/mpi/kubexec.sh"

_RANK_SIZE_VARS = (("HOROVOD_RANK", "HOROVOD_SIZE"),
                   ("OMPI_COMM_WORLD_RANK", "OMPI_COMM_WORLD_SIZE"),
                   ("PMI_RANK", "PMI_SIZE"))


def is_exportable(name):
    return not any(re.match(pattern, name) for pattern in IGNORE_REGEXES)


def get_env_rank_and_size():
    """(rank, size) from the first launcher whose pair of variables is set;
    (0, 1) when none is. Half a pair is an error."""
    for rank_var, size_var in _RANK_SIZE_VARS:
        rank, size = os.environ.get(rank_var), os.environ.get(size_var)
        if rank is not None and size is not None:
            return int(rank), int(size)
        if (rank is None) != (size is None):
            raise RuntimeError("Could not determine process rank and size: only one of %s and "
                               "%s found in environment" % (rank_var, size_var))
    return 0, 1


def is_kubeflow_mpi():
    return os.environ.get("OMPI_MCA_plm_rsh_agent") == KUBEFLOW_MPI_EXEC
